from .job_config import FaultTolerance

__all__ = ["FaultTolerance"]
