"""oslo_b200: a Blackwell-native (sm_100a) 3D-parallel transformer training / inference framework.

Public surface mirrors the reference package (oslo/__init__.py:3-17): models, configs, data
classes, the parallel layers and ``oslo_b200.parallelize``.
"""
import os as _os

# A pipeline stage keeps receives posted on their own streams while it computes. With more streams than hardware work
# queues (8 by default) two streams can share a queue, and a receive that waits for its sender would then hold up
# the very computation the sender is waiting for. The variable is read when the CUDA context is created.
_os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")
# Point-to-point transfers between pipeline stages: two channels (two thread blocks per transfer kernel) are enough for
# one activation per micro-batch over NVLink, and every block of a transfer that waits for its peer holds an SM.
_os.environ.setdefault("NCCL_MAX_P2P_NCHANNELS", "2")

# Load every kernel when the CUDA context is created instead of at its first launch (costs about a second and 0.6 GB).
# A first launch that has to load its kernel can wait for all kernels running in the context; under pipeline
# parallelism one of those may be a transfer that waits for the neighbouring stage, which in turn waits for this
# process to get further - the lazy default turns that into a deadlock in the first step.
_os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")

from .__version__ import version as __version__  # noqa: F401,E402
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
