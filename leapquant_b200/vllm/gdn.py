"""LeapQuant on the engine's Gated DeltaNet layers (the role of reference leapquant/vllm/gdn.py:11-81).

`GdnAdapter` carries out the plan of routing.plan_gdn_step with the engine's tensors; `install()` builds one from the
installed vLLM and puts it in place of QwenGatedDeltaNetAttention's core forward and of the module-level decode kernel
the engine calls for the decode tokens of a mixed step.  The engine-side names the adapter needs are looked up once, so
that one adapter serves the vLLM the reference pins (0.30: `_forward_core`, metadata with `prefill_state_indices`) and the
older layout this package is also tested with (0.22: no `prefill_state_indices`, where a mixed step falls back to the
round trip of every touched slot).
"""
import torch

from ..state import get_state
from .routing import Route, conv_weight_2d, layer_metadata, plan_gdn_step


class GdnAdapter:
    def __init__(self, module, nmax, get_forward_context, causal_conv1d_update, conv_state_dim_first):
        self.module = module                                  # the engine module that holds the layer class and its decode kernel
        self.cls = module.QwenGatedDeltaNetAttention
        self.nmax = nmax
        self.get_forward_context = get_forward_context
        self.conv_update = causal_conv1d_update
        self.conv_state_dim_first = conv_state_dim_first
        self.core_name = "_forward_core" if hasattr(self.cls, "_forward_core") else "forward_core"
        self.engine_core = getattr(self.cls, self.core_name)
        self.engine_decode_kernel = getattr(module, "fused_sigmoid_gating_delta_rule_update", None)
        self.mixed_layer = None                               # the layer whose MIXED step is inside the engine's forward right now
        self.fuse_conv = True                                 # pure decode: conv1d update and decode through state.decode_conv()

    # ---- pieces ----
    def state_of(self, layer):
        return get_state(layer, layer.kv_cache[1], H=layer.num_k_heads // layer.tp_size, nmax=self.nmax[0])

    def decode_tokens(self, layer, mixed_qkv, b, a, core_attn_out, md):
        """DECODE route: the conv1d update of the n live rows, then one decode call on the 8-bit state."""
        n = md.num_actual_tokens
        slots = md.non_spec_state_indices_tensor[:n]
        conv_cache, ssm = layer.kv_cache[0], layer.kv_cache[1]
        conv_state = conv_cache if self.conv_state_dim_first() else conv_cache.transpose(-1, -2)
        if self.fuse_conv and layer.activation in ("silu", "swish") and mixed_qkv.dtype == torch.bfloat16:
            # conv1d update, step and flush as ONE launch: the activated q | k | v row never goes through memory
            st = self.state_of(layer)
            st.decode_conv(ssm, mixed_qkv[:n], conv_state, conv_weight_2d(layer.conv1d), layer.conv1d.bias, a[:n].contiguous(),
                           b[:n].contiguous(), layer.A_log, layer.dt_bias, slots, core_attn_out[:n].view(n, st.HV, st.V))
            return
        mixed = self.conv_update(mixed_qkv[:n], conv_state, conv_weight_2d(layer.conv1d), layer.conv1d.bias, layer.activation,
                                 conv_state_indices=slots, validate_data=False)
        st = self.state_of(layer)
        st.decode(ssm, mixed.contiguous(), a[:n].contiguous(), b[:n].contiguous(), layer.A_log, layer.dt_bias, slots,
                  core_attn_out[:n].view(n, st.HV, st.V))

    def decode_kernel(self, A_log, a, b, dt_bias, q, k, v, initial_state, inplace_final_state, cu_seqlens, ssm_state_indices,
                      use_qk_l2norm_in_kernel=True, **kw):
        """Stands in for the engine's fused decode kernel.  While a MIXED step of one of our layers is inside the engine's
        forward, the single-token call it makes for the step's decode tokens runs on the 8-bit state instead; every other
        call (another layer type, speculative verification, multi-token) goes to the engine's kernel untouched."""
        layer = self.mixed_layer
        if layer is None or kw.get("num_accepted_tokens") is not None or q.shape[0] != 1:
            return self.engine_decode_kernel(A_log=A_log, a=a, b=b, dt_bias=dt_bias, q=q, k=k, v=v, initial_state=initial_state,
                                             inplace_final_state=inplace_final_state, cu_seqlens=cu_seqlens,
                                             ssm_state_indices=ssm_state_indices,
                                             use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel, **kw)
        st = self.state_of(layer)
        n = q.shape[1]
        rows = [t.reshape(n, -1) for t in (q, k, v)]
        mixed = torch.cat(rows, dim=1).to(torch.bfloat16).contiguous()
        out = torch.empty(n, st.HV, st.V, dtype=torch.bfloat16, device=q.device)
        st.decode(layer.kv_cache[1], mixed, a[:n].contiguous(), b[:n].contiguous(), A_log, dt_bias, ssm_state_indices[:n], out)
        return out.unsqueeze(0), None

    def forward_core(self, layer, mixed_qkv, b, a, core_attn_out):
        md = layer_metadata(self.get_forward_context(), layer.prefix)
        plan = plan_gdn_step(md, getattr(layer, "enable_packed_recurrent_decode", True))
        if md is None:
            return self.engine_core(layer, mixed_qkv, b, a, core_attn_out)
        if plan.route is Route.DECODE:
            return self.decode_tokens(layer, mixed_qkv, b, a, core_attn_out, md)
        st = self.state_of(layer)                             # (created on the layer's first step that is not a pure decode)
        if plan.route is Route.ENGINE:                        # the step touches no state slot
            return self.engine_core(layer, mixed_qkv, b, a, core_attn_out)
        ssm = layer.kv_cache[1]
        st.dequantize(ssm, plan.slots)
        reroute = plan.route is Route.MIXED and self.engine_decode_kernel is not None
        self.mixed_layer = layer if reroute else None
        try:
            ret = self.engine_core(layer, mixed_qkv, b, a, core_attn_out)
        finally:
            self.mixed_layer = None
        st.quantize(ssm, plan.slots)
        return ret

    # ---- wiring ----
    def patch(self):
        adapter = self
        if self.engine_decode_kernel is not None:
            self.module.fused_sigmoid_gating_delta_rule_update = self.decode_kernel
        setattr(self.cls, self.core_name,
                lambda layer, mixed_qkv, b, a, core_attn_out: adapter.forward_core(layer, mixed_qkv, b, a, core_attn_out))
        return self


def install(nmax):
    from vllm.forward_context import get_forward_context
    from vllm.model_executor.layers.mamba.gdn import qwen_gdn_linear_attn as module
    from vllm.model_executor.layers.mamba.ops.causal_conv1d import causal_conv1d_update
    try:
        from vllm.model_executor.layers.mamba.mamba_utils import is_conv_state_dim_first
    except ImportError:                                   # layouts that predate the switch keep the conv state dim-first
        def is_conv_state_dim_first():
            return True
    return GdnAdapter(module, nmax, get_forward_context, causal_conv1d_update, is_conv_state_dim_first).patch()
