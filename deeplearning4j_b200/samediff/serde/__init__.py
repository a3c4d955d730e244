"""SameDiff serialisation: FlatBuffers FlatGraph (``.fb``), SDNB containers and SDZ archives."""
from .flatgraph import from_flatbuffers, to_flatbuffers  # noqa: F401
from .sdnb import load, load_sdz, save, save_sdz  # noqa: F401
