"""LeapQuant on vLLM's GLM Kimi-Delta-Attention layers (reference leapquant/vllm/glm.py:12-77).

Pure decode steps run the KDA step + flush kernels on the 8-bit state.  In steps with prefill tokens the decode tokens go
through the quantized path first and only the prefill slots take an fp32 round trip around vLLM's own prefill kernel.
The replaced forward stays an eager break of vLLM's breakable CUDA graph.
"""
import torch

from ..state import get_state


def install(nmax):
    from vllm.compilation.breakable_cudagraph import eager_break_during_capture
    from vllm.forward_context import get_forward_context
    from vllm.model_executor.layers.mamba.ops.causal_conv1d import causal_conv1d_update
    from vllm.models.glm5next.nvidia import kda as KM

    cls = KM.Glm5NextLinearAttention
    orig = getattr(cls._forward, "__wrapped__", cls._forward)

    def layer_state(layer):
        return get_state(layer, layer.kv_cache[1], H=layer.local_num_heads, kda=True,
                         gate_lower_bound=float(layer.kda_lower_bound), nmax=nmax[0])

    def merged_conv_weight(layer):
        if layer._merged_conv_weight is None:
            flat = [m.weight.view(m.weight.size(0), m.weight.size(2)) for m in (layer.q_conv1d, layer.k_conv1d, layer.v_conv1d)]
            layer._merged_conv_weight = torch.cat(flat, dim=0).contiguous()
        return layer._merged_conv_weight

    def forward(layer, qkv_proj_states, g1, beta, core_attn_out):
        md_all = get_forward_context().attn_metadata
        m = md_all.get(layer.prefix) if isinstance(md_all, dict) else None
        if m is None or m.num_actual_tokens == 0:
            return
        n = m.num_actual_tokens
        assert layer.kda_safe_gate and layer.kda_lower_bound is not None, "LeapQuant supports the bounded KDA gate only"
        st = layer_state(layer)
        kv = layer.kv_cache
        if m.spec_sequence_masks is not None and m.num_spec_decodes > 0:       # speculative decoding: round trip every slot
            parts = [t.reshape(-1) for t in (m.non_spec_state_indices_tensor, m.spec_state_indices_tensor) if t is not None]
            touched = torch.cat(parts).clamp(min=0)
            st.dequantize(kv[1], touched)
            orig(layer, qkv_proj_states=qkv_proj_states, g1=g1, beta=beta, core_attn_out=core_attn_out)
            st.quantize(kv[1], touched)
            return
        conv_state = kv[0] if layer._conv_state_dim_first else kv[0].transpose(-1, -2)
        wconv = merged_conv_weight(layer)
        if m.num_prefills > 0:
            nd = m.num_decode_tokens
            slots = m.non_spec_state_indices_tensor
            x = KM.causal_conv1d_fn(qkv_proj_states[:n].transpose(0, 1), wconv, layer.q_conv1d.bias, activation="silu",
                                    conv_states=conv_state, has_initial_state=m.has_initial_state, cache_indices=slots,
                                    query_start_loc=m.non_spec_query_start_loc, metadata=m).transpose(0, 1)
            if nd > 0:                                   # decode tokens first, through the quantized path
                st.decode(kv[1], x[:nd].contiguous(), g1[0, :nd], beta[0, :nd].contiguous(), layer.A_log.view(-1),
                          layer.dt_bias, slots[:nd], core_attn_out[0, :nd])
            pslots, phas, ploc = m.prefill_state_indices, m.prefill_has_initial_state, m.prefill_query_start_loc
            st.dequantize(kv[1], pslots.clamp(min=0))    # fp32 state for the prefill slots only
            init = KM.gather_initial_states(kv[1], pslots, phas)
            heads = lambda t: t.reshape(1, -1, layer.local_num_heads, layer.head_dim)
            q, k, v = (heads(t) for t in x[nd:n].split(layer.local_projection_size, dim=-1))
            if layer.kda_prefill_backend == "flashkda":
                outp, last = layer._flashkda_prefill(q=q, k=k, v=v, g=g1[:, nd:n], beta=beta[:, nd:n], initial_state=init,
                                                     cu_seqlens=ploc, out=None)
            else:
                outp, last = KM.chunk_kda_with_fused_gate(
                    q=q, k=k, v=v, raw_g=g1[:, nd:n], beta=KM._cast_sigmoid(beta[:, nd:n].squeeze(0)).unsqueeze(0),
                    A_log=layer.A_log, g_bias=layer.dt_bias, initial_state=init, output_final_state=True,
                    use_qk_l2norm_in_kernel=True, cu_seqlens=ploc, safe_gate=layer.kda_safe_gate,
                    lower_bound=layer.kda_lower_bound)
            KM.scatter_states(kv[1], last, pslots)
            core_attn_out[0, nd:n] = outp[0, :n - nd]
            st.quantize(kv[1], pslots.clamp(min=0))      # checkpoint written when the prefill ends
            return
        slots = m.non_spec_state_indices_tensor[:n]
        mixed = causal_conv1d_update(qkv_proj_states[:n], conv_state, wconv, layer.q_conv1d.bias, activation="silu",
                                     conv_state_indices=slots)
        st.decode(kv[1], mixed.contiguous(), g1[0, :n], beta[0, :n].contiguous(), layer.A_log.view(-1), layer.dt_bias,
                  slots, core_attn_out[0, :n])

    cls._forward = eager_break_during_capture(forward)
