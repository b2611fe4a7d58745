from .logging import get_logger  # noqa: F401
from .metrics import MetricsLogger, load_measured_peaks, roofline_fraction, transformer_train_flops  # noqa: F401
from .timers import DeviceTimer, nvtx_range  # noqa: F401
from .watchdog import Heartbeat, OsloCommTimeout, RankFailure, StepDeadline, raise_if_device_error  # noqa: F401
from .checkpoint import (CheckpointManager, CheckpointUnreadable, atomic_save, load_training_state,  # noqa: F401
                         save_training_state, state_file)
