from .calibrator import AMaxCalibrator, BaseCalibrator, CalibratorRegistry  # noqa: F401
