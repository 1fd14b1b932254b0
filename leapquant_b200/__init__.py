"""leapquant_b200: LeapQuant's quantized recurrent-state decode path for linear attention (GDN / KDA), rebuilt for
NVIDIA B200 (sm_100a) as hand-written CUDA kernels behind a C ABI, with the reference's Python API on top.

    leapquant_b200.state     LeapQuantState, state_views, get_state, WINDOW, RANK   (reference leapquant/state.py)
    leapquant_b200.kernels   make_gdn_step / make_kda_step / make_flush / make_dequant / make_quantize / make_lowrank
                             (reference leapquant/kernels.py)
    leapquant_b200.vllm      register(), gdn.install(), glm.install()               (reference leapquant/vllm/)

`install_alias()` publishes the package under the name `leapquant`, so code written against the reference
(`from leapquant.state import get_state`) runs on these kernels without edits.
"""
import sys

__version__ = "0.1.0"


def install_alias(name="leapquant"):
    """Register this package (and its state / kernels / vllm modules) in sys.modules under `name`."""
    import importlib
    pkg = sys.modules[__name__]
    sys.modules.setdefault(name, pkg)
    for sub in ("state", "kernels", "vllm"):
        sys.modules.setdefault(f"{name}.{sub}", importlib.import_module(f"{__name__}.{sub}"))
    return pkg
