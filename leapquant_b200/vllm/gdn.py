"""LeapQuant on vLLM's Gated DeltaNet layers (reference leapquant/vllm/gdn.py:11-81).

Routing, unchanged from the reference: a pure decode step runs the step + flush kernels on the 8-bit state; in a step
that also carries prefill tokens the decode tokens still go through the quantized path and only the prefill slots take
an fp32 round trip (dequantize -> vLLM's chunked prefill -> quantize); speculative decoding round-trips every slot.
"""
import torch

from ..state import get_state


def install(nmax):
    from vllm.forward_context import get_forward_context
    from vllm.model_executor.layers.mamba.gdn import qwen_gdn_linear_attn as M
    from vllm.model_executor.layers.mamba.ops.causal_conv1d import causal_conv1d_update
    try:
        from vllm.model_executor.layers.mamba.mamba_utils import is_conv_state_dim_first
    except ImportError:                                   # older layouts keep the conv state dim-first
        def is_conv_state_dim_first():
            return True

    cls = M.QwenGatedDeltaNetAttention
    core_name = "_forward_core" if hasattr(cls, "_forward_core") else "forward_core"
    orig_core = getattr(cls, core_name)
    orig_fsg = getattr(M, "fused_sigmoid_gating_delta_rule_update", None)
    active = [None]                    # the layer whose mixed prefill + decode step is running

    def layer_state(layer):
        return get_state(layer, layer.kv_cache[1], H=layer.num_k_heads // layer.tp_size, nmax=nmax[0])

    def run_decode(layer, mixed_qkv, b, a, core_attn_out, md):
        slots = md.non_spec_state_indices_tensor
        kv = layer.kv_cache
        conv_state = kv[0] if is_conv_state_dim_first() else kv[0].transpose(-1, -2)
        n = md.num_actual_tokens
        w = layer.conv1d.weight
        mixed = causal_conv1d_update(mixed_qkv[:n], conv_state, w.view(w.size(0), w.size(2)), layer.conv1d.bias,
                                     layer.activation, conv_state_indices=slots[:n], validate_data=False)
        st = layer_state(layer)
        st.decode(kv[1], mixed.contiguous(), a[:n].contiguous(), b[:n].contiguous(), layer.A_log, layer.dt_bias,
                  slots[:n], core_attn_out[:n].view(n, st.HV, st.V))

    def routed_fsg(A_log, a, b, dt_bias, q, k, v, initial_state, inplace_final_state, cu_seqlens, ssm_state_indices,
                   use_qk_l2norm_in_kernel=True, **kw):
        """vLLM's own decode kernel, called for the decode tokens inside a mixed step, redirected to the step kernel."""
        layer = active[0]
        if layer is None or kw.get("num_accepted_tokens") is not None or q.shape[0] != 1:
            return orig_fsg(A_log=A_log, a=a, b=b, dt_bias=dt_bias, q=q, k=k, v=v, initial_state=initial_state,
                            inplace_final_state=inplace_final_state, cu_seqlens=cu_seqlens,
                            ssm_state_indices=ssm_state_indices, use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel, **kw)
        st = layer_state(layer)
        n = q.shape[1]
        mixed = torch.cat([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], dim=1).to(torch.bfloat16).contiguous()
        out = torch.empty(n, st.HV, st.V, dtype=torch.bfloat16, device=q.device)
        st.decode(layer.kv_cache[1], mixed, a[:n].contiguous(), b[:n].contiguous(), A_log, dt_bias,
                  ssm_state_indices[:n], out)
        return out.unsqueeze(0), None

    def forward_core(layer, mixed_qkv, b, a, core_attn_out):
        md_all = get_forward_context().attn_metadata
        md = md_all.get(layer.prefix) if isinstance(md_all, dict) else None
        if md is None:                                   # profiling / warm-up runs
            return orig_core(layer, mixed_qkv, b, a, core_attn_out)
        packed = getattr(layer, "enable_packed_recurrent_decode", True)
        if packed and md.spec_sequence_masks is None and md.num_prefills == 0 and md.num_decodes > 0:
            return run_decode(layer, mixed_qkv, b, a, core_attn_out, md)
        st = layer_state(layer)
        prefill_slots = getattr(md, "prefill_state_indices", None)
        if md.spec_sequence_masks is None and prefill_slots is not None:
            touched = prefill_slots.reshape(-1).clamp(min=0)                # prefill slots only
            route = True
        else:                                                               # speculative decoding: round trip every slot
            parts = [t.reshape(-1) for t in (md.non_spec_state_indices_tensor, md.spec_state_indices_tensor)
                     if t is not None]
            if not parts:
                return orig_core(layer, mixed_qkv, b, a, core_attn_out)
            touched = torch.cat(parts).clamp_(min=0)
            route = False
        st.dequantize(layer.kv_cache[1], touched)
        active[0] = layer if (route and orig_fsg is not None) else None
        try:
            ret = orig_core(layer, mixed_qkv, b, a, core_attn_out)
        finally:
            active[0] = None
        st.quantize(layer.kv_cache[1], touched)
        return ret

    if orig_fsg is not None:
        M.fused_sigmoid_gating_delta_rule_update = routed_fsg
    setattr(cls, core_name, forward_core)
