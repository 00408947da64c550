"""B200 (sm_100a) 1-D neighbourhood attention behind the PCF-NAT ``nattn.py`` interface."""
from .nattn import getNA1dFunction, install_as_na1d_tensorcore  # noqa: F401
from .ops import NA1dFusedFunction, fused_forward, fused_backward, window_index  # noqa: F401
from .library_op import na1d_fused  # noqa: F401
from .nattention import GlobalAttention, NAttention, fuse_nattention  # noqa: F401

__all__ = ["getNA1dFunction", "install_as_na1d_tensorcore", "na1d_fused", "NA1dFusedFunction",
           "fused_forward", "fused_backward", "window_index", "NAttention", "GlobalAttention", "fuse_nattention"]
