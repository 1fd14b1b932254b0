"""vLLM integration: once registered, the recurrent states of GDN (Qwen) and KDA (GLM) layers are kept in 8 bits.

Mirrors the reference's leapquant/vllm/__init__.py:8-34.  The entry point is `leapquant_b200.vllm:register`
(group `vllm.general_plugins`).  A layer class that this vLLM build does not ship is skipped with a message
instead of failing the whole registration, so the GDN path installs on builds without the GLM KDA layer.
"""
import importlib
import os

_INSTALLED = []
_NMAX = [0]          # largest decode batch one call can carry


def _record_nmax(cls):
    """Wrap the layer constructor to record max_num_seqs / the CUDA-graph capture size of the vLLM config being built."""
    init = cls.__init__

    def __init__(self, *a, **k):
        init(self, *a, **k)
        from vllm.config import get_current_vllm_config
        cfg = get_current_vllm_config()
        cc = cfg.compilation_config
        _NMAX[0] = max(_NMAX[0], cfg.scheduler_config.max_num_seqs, getattr(cc, "max_cudagraph_capture_size", None) or 0)

    cls.__init__ = __init__


def _try(modname, attr):
    try:
        return getattr(importlib.import_module(modname), attr)
    except (ImportError, AttributeError):
        return None


def register():
    """vllm.general_plugins entry point, run in every vLLM process."""
    if _INSTALLED:
        return
    from . import gdn, glm
    done = []
    gdn_cls = _try("vllm.model_executor.layers.mamba.gdn.qwen_gdn_linear_attn", "QwenGatedDeltaNetAttention")
    if gdn_cls is not None:
        _record_nmax(gdn_cls)
        gdn.install(_NMAX)
        done.append("GDN")
    kda_cls = _try("vllm.models.glm5next.nvidia.kda", "Glm5NextLinearAttention")
    if kda_cls is not None:
        _record_nmax(kda_cls)
        glm.install(_NMAX)
        done.append("KDA")
    _INSTALLED.append(True)
    print(f"[LeapQuant-B200] 8-bit recurrent states enabled for {'+'.join(done) or 'no layer class found'} "
          f"(pid {os.getpid()})", flush=True)
