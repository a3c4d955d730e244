"""Runtime utilities: workspaces, environment flags, profiler / executioner, compression SPI."""
from .environment import Environment, ND4JEnvironmentVars, ND4JSystemProperties  # noqa: F401
from .workspace import (AllocationPolicy, BasicWorkspaceManager, LearningPolicy, MemoryWorkspace, ResetPolicy, SpillPolicy,  # noqa: F401
                        WorkspaceConfiguration, WorkspaceMgr, getWorkspaceManager)
