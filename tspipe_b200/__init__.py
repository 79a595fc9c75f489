"""tspipe_b200: a Blackwell-native teacher-student pipeline training runtime."""
from .__version__ import __version__
from .batch_ops import Batch, BatchQueue, ScatterGatherFn, defaultScatterGatherFn, gather, scatter
from .batchnorm import DeferredBatchNorm
from .model_wrapper import TSPipeModelOutput, TSPipeModelWrapper
from .tspipe import BalanceError, TSPipe, TSPipeMode

__all__ = ["TSPipe", "TSPipeMode", "BalanceError", "TSPipeModelWrapper", "TSPipeModelOutput", "ScatterGatherFn",
           "defaultScatterGatherFn", "DeferredBatchNorm", "Batch", "BatchQueue", "scatter", "gather",
           "__version__"]
