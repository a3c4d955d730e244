"""DL4J neural-network API: configurations, layers, MultiLayerNetwork / ComputationGraph,
updaters and ModelSerializer."""
from .activations import Activation
from .losses import LossFunctions
from .weights import WeightInit
from .updaters import (Sgd, Nesterovs, Adam, AdaMax, Nadam, AMSGrad, AdaBelief, AdaGrad, AdaDelta, RmsProp, NoOp,
                       ScheduleType, FixedSchedule, ExponentialSchedule, InverseSchedule, MapSchedule, PolySchedule,
                       SigmoidSchedule, StepSchedule, RampSchedule, CycleSchedule,
                       L1Regularization, L2Regularization, WeightDecay)
from .conf.base import (InputType, ConvolutionMode, PoolingType, BackpropType, GradientNormalization, WorkspaceMode,
                        CacheMode, CNN2DFormat, RNNFormat, Dropout, SpatialDropout, AlphaDropout, GaussianDropout,
                        GaussianNoise, MaxNormConstraint, MinMaxNormConstraint, NonNegativeConstraint,
                        UnitNormConstraint, DropConnect, WeightNoise)
from .conf.neuralnet import NeuralNetConfiguration, MultiLayerConfiguration
from .layers.core import *      # noqa: F401,F403
from .layers.conv import *      # noqa: F401,F403
from .layers.recurrent import *  # noqa: F401,F403
from .layers.attention import *  # noqa: F401,F403
from .layers.special import *  # noqa: F401,F403
from .multilayer import MultiLayerNetwork
from .serializer import ModelSerializer, ModelGuesser
from .graph import ComputationGraph  # noqa: E402
from .conf.graphconf import (ComputationGraphConfiguration, ElementWiseVertex, MergeVertex, SubsetVertex, StackVertex,  # noqa: E402
                             UnstackVertex, ScaleVertex, ShiftVertex, L2NormalizeVertex, L2Vertex, ReshapeVertex,
                             PreprocessorVertex, PoolHelperVertex, FrozenVertex, LayerVertex)
from .earlystopping import (EarlyStoppingConfiguration, EarlyStoppingTrainer, EarlyStoppingGraphTrainer,  # noqa: E402
                            EarlyStoppingResult)
from .transferlearning import FineTuneConfiguration, TransferLearning, TransferLearningHelper  # noqa: E402
