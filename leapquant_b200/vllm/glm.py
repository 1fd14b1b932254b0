"""LeapQuant on the engine's GLM Kimi-Delta-Attention layers (the role of reference leapquant/vllm/glm.py:12-77).

`KdaAdapter` carries out the plan of routing.plan_kda_step.  Unlike the Gated DeltaNet layer, the engine's KDA forward
cannot be wrapped for a mixed step: its prefill kernel takes the initial states as an argument, so the adapter runs the
pieces itself -- conv over all tokens, the decode tokens on the 8-bit state, then dequantize -> gather -> the engine's
chunked KDA prefill -> scatter -> quantize for the prefill slots.  The replaced forward stays an eager break of the
engine's breakable CUDA graph, as in the reference.
"""
import torch

from ..state import get_state
from .routing import Route, conv_weight_2d, layer_metadata, plan_kda_step


class KdaAdapter:
    def __init__(self, module, nmax, get_forward_context, causal_conv1d_update, eager_break):
        self.module = module                                  # engine module: layer class + prefill helpers
        self.cls = module.Glm5NextLinearAttention
        self.nmax = nmax
        self.get_forward_context = get_forward_context
        self.conv_update = causal_conv1d_update
        self.eager_break = eager_break
        self.engine_forward = getattr(self.cls._forward, "__wrapped__", self.cls._forward)
        self.fuse_conv = True                                 # pure decode: conv1d update and decode through state.decode_conv()

    def state_of(self, layer):
        return get_state(layer, layer.kv_cache[1], H=layer.local_num_heads, kda=True,
                         gate_lower_bound=float(layer.kda_lower_bound), nmax=self.nmax[0])

    @staticmethod
    def conv_operands(layer):
        """The conv state in (slot, dim, width - 1) order and the q | k | v depthwise weights as one [dim, width] matrix
        (built once per layer and kept where the engine's own forward keeps it)."""
        cache = layer.kv_cache[0]
        conv_state = cache if layer._conv_state_dim_first else cache.transpose(-1, -2)
        if layer._merged_conv_weight is None:
            parts = [conv_weight_2d(m) for m in (layer.q_conv1d, layer.k_conv1d, layer.v_conv1d)]
            layer._merged_conv_weight = torch.cat(parts, dim=0).contiguous()
        return conv_state, layer._merged_conv_weight

    def prefill_slots(self, layer, st, m, x, g1, beta, core_attn_out, nd, n):
        """fp32 round trip of the prefill slots around the engine's chunked KDA prefill, tokens nd .. n-1."""
        KM, ssm = self.module, layer.kv_cache[1]
        slots = m.prefill_state_indices
        live = slots.clamp(min=0)
        st.dequantize(ssm, live)
        init = KM.gather_initial_states(ssm, slots, m.prefill_has_initial_state)
        q, k, v = (t.reshape(1, -1, layer.local_num_heads, layer.head_dim)
                   for t in x[nd:n].split(layer.local_projection_size, dim=-1))
        if layer.kda_prefill_backend == "flashkda":
            outp, last = layer._flashkda_prefill(q=q, k=k, v=v, g=g1[:, nd:n], beta=beta[:, nd:n], initial_state=init,
                                                 cu_seqlens=m.prefill_query_start_loc, out=None)
        else:
            outp, last = KM.chunk_kda_with_fused_gate(
                q=q, k=k, v=v, raw_g=g1[:, nd:n], beta=KM._cast_sigmoid(beta[:, nd:n].squeeze(0)).unsqueeze(0),
                A_log=layer.A_log, g_bias=layer.dt_bias, initial_state=init, output_final_state=True,
                use_qk_l2norm_in_kernel=True, cu_seqlens=m.prefill_query_start_loc, safe_gate=layer.kda_safe_gate,
                lower_bound=layer.kda_lower_bound)
        KM.scatter_states(ssm, last, slots)
        core_attn_out[0, nd:n] = outp[0, :n - nd]
        st.quantize(ssm, live)

    def forward(self, layer, qkv_proj_states, g1, beta, core_attn_out):
        m = layer_metadata(self.get_forward_context(), layer.prefix)
        plan = plan_kda_step(m)
        if plan.route is Route.ENGINE:
            return
        assert layer.kda_safe_gate and layer.kda_lower_bound is not None, "LeapQuant supports the bounded KDA gate only"
        st = self.state_of(layer)
        ssm = layer.kv_cache[1]
        n = m.num_actual_tokens
        if plan.route is Route.ROUND_TRIP:
            st.dequantize(ssm, plan.slots)
            self.engine_forward(layer, qkv_proj_states=qkv_proj_states, g1=g1, beta=beta, core_attn_out=core_attn_out)
            st.quantize(ssm, plan.slots)
            return
        conv_state, wconv = self.conv_operands(layer)
        decode = lambda rows, cnt, slots: st.decode(ssm, rows.contiguous(), g1[0, :cnt], beta[0, :cnt].contiguous(),
                                                    layer.A_log.view(-1), layer.dt_bias, slots, core_attn_out[0, :cnt])
        if plan.route is Route.DECODE:
            slots = m.non_spec_state_indices_tensor[:n]
            if self.fuse_conv and qkv_proj_states.dtype == torch.bfloat16:
                st.decode_conv(ssm, qkv_proj_states[:n], conv_state, wconv, layer.q_conv1d.bias, g1[0, :n], beta[0, :n].contiguous(),
                               layer.A_log.view(-1), layer.dt_bias, slots, core_attn_out[0, :n])
                return
            mixed = self.conv_update(qkv_proj_states[:n], conv_state, wconv, layer.q_conv1d.bias, activation="silu",
                                     conv_state_indices=slots)
            decode(mixed, n, slots)
            return
        # MIXED: one conv over all tokens, the decode tokens (they come first) on the 8-bit state, then the prefill slots
        nd = m.num_decode_tokens
        slots = m.non_spec_state_indices_tensor
        x = self.module.causal_conv1d_fn(qkv_proj_states[:n].transpose(0, 1), wconv, layer.q_conv1d.bias, activation="silu",
                                         conv_states=conv_state, has_initial_state=m.has_initial_state, cache_indices=slots,
                                         query_start_loc=m.non_spec_query_start_loc, metadata=m).transpose(0, 1)
        if nd > 0:
            decode(x[:nd], nd, slots[:nd])
        self.prefill_slots(layer, st, m, x, g1, beta, core_attn_out, nd, n)

    def patch(self):
        adapter = self
        self.cls._forward = self.eager_break(
            lambda layer, qkv_proj_states, g1, beta, core_attn_out: adapter.forward(layer, qkv_proj_states, g1, beta, core_attn_out))
        return self


def install(nmax):
    from vllm.compilation.breakable_cudagraph import eager_break_during_capture
    from vllm.forward_context import get_forward_context
    from vllm.model_executor.layers.mamba.ops.causal_conv1d import causal_conv1d_update
    from vllm.models.glm5next.nvidia import kda as module
    return KdaAdapter(module, nmax, get_forward_context, causal_conv1d_update, eager_break_during_capture).patch()
