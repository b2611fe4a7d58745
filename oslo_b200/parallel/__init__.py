from .mpu import MPU, Layer, LayerPolicy  # noqa: F401
