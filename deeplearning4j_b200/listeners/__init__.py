"""Training listeners for MultiLayerNetwork / ComputationGraph (SameDiff listeners: ``samediff.listeners``)."""
from .training import *  # noqa: F401,F403
from .training import TrainingListener, BaseTrainingListener  # noqa: F401
