from .tileop import builtin, cuda_link, hip_link, triton_fn

__all__ = ["builtin", "cuda_link", "hip_link", "triton_fn"]
