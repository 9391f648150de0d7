"""B200-native microscaling attention: flash_attn_fp8 (MXFP8) and flash_attn_fp4 (mixed NVFP4 / FP8), forward and
backward, behind the public interface of the reference's flash_attn.cute.lowprec package (entry points, option objects,
plan resolution, torch custom ops). The compute path is hand-written CUDA for sm_100a in libflamia_b200.so, reached
through the C ABI of include/flamia_b200.h; there is no CPU or PyTorch fallback.
"""
from .docmaps import DocMaps
from .options import FP4AttnOptions, FP8AttnOptions, KernelTuning, TUNING_FIELDS
from .plan import AttnPlan, resolve_fp4, resolve_fp8

__all__ = ["flash_attn_fp4", "flash_attn_fp8", "check_status", "DocMaps", "FP4AttnOptions", "FP8AttnOptions", "KernelTuning", "TUNING_FIELDS",
           "AttnPlan", "resolve_fp4", "resolve_fp8"]


def __getattr__(name):
    # the entry points import torch.library ops and the C-ABI loader: resolved on first use so that the option / plan
    # modules import on a machine without the built library
    if name in ("flash_attn_fp4", "flash_attn_fp8"):
        from . import api
        return getattr(api, name)
    if name == "check_status":
        from ._routes import check_status
        return check_status
    raise AttributeError(name)
