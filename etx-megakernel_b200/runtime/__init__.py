from .lib import BODY, EtxbError, StepParams, build, check, device_info, load
from .session import Session, op_launch

__all__ = ["BODY", "EtxbError", "StepParams", "build", "check", "device_info", "load", "Session", "op_launch"]
