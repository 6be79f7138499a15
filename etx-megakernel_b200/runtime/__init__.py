from .lib import BODY, EtxbError, StepParams, build, check, device_info, load
from .session import ExchangeRegion, Session, attn_fused_static, op_launch

__all__ = ["BODY", "EtxbError", "StepParams", "build", "check", "device_info", "load", "ExchangeRegion", "Session", "attn_fused_static", "op_launch"]
