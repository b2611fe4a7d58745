"""oslo_b200: a Blackwell-native (sm_100a) 3D-parallel transformer training / inference framework.

Public surface mirrors the reference package (oslo/__init__.py:3-17): models, configs, data
classes, the parallel layers and ``oslo_b200.parallelize``.
"""
from .__version__ import version as __version__  # noqa: F401
from .modeling_utils import *  # noqa: F401,F403
from .modeling_utils import PreTrainedModel, PretrainedConfig, ModelOutput  # noqa: F401
from .parallel.mpu import MPU, Layer, LayerPolicy  # noqa: F401
from .parallel.layers import (ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding,  # noqa: F401
                              Linear, Conv1D, LayerNorm, Embedding)
from .parallelism_utils import ParallelizationMixin  # noqa: F401
from .fused_kernels_utils import (FusedKernelMixin, FusedScaleMaskSoftmax, FusedBiasActivation,  # noqa: F401
                                  FusedBiasDropout, FusedBiasDropoutResidual, get_custom_kernels,
                                  get_datasets_builder)
from .generation import *  # noqa: F401,F403
from .models import *  # noqa: F401,F403
from .data import *  # noqa: F401,F403
from .optim import FusedAdamW  # noqa: F401

parallelize = ParallelizationMixin._parallelize_from_model
