"""CPU tests of the serving-engine plugin (leapquant_b200.vllm) against stub `vllm` modules.

The stubs stand in for the engine classes and kernels the plugin patches or calls (the layer classes, the forward context,
the conv1d kernels, the engine's own decode and prefill kernels); a recording object stands in for LeapQuantState.  Every
scenario drives one patched layer forward and records, in order, what was called with which slots and shapes:

  * Gated DeltaNet: warm-up without metadata, pure decode, mixed prefill + decode with the engine's decode kernel rerouted,
    speculative decoding (round trip of every touched slot), and an engine whose metadata has no separate prefill slots;
  * Kimi Delta Attention: empty step, pure decode, mixed prefill + decode, speculative decoding.

Where the reference checkout is present the same scenarios are driven through the REFERENCE'S OWN plugin files
(leapquant/vllm/gdn.py, leapquant/vllm/glm.py), loaded from the checkout and bound to this package through
`install_alias()`, and the two call logs must be identical.
"""
import importlib
import importlib.util
import os
import sys
import types

import pytest
import torch

# a checkout of the reference: LEAPQUANT_REFERENCE, or a directory `reference` beside this repository
REF = os.environ.get("LEAPQUANT_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
HAVE_REF = os.path.exists(os.path.join(REF, "leapquant", "vllm", "gdn.py"))
NS = types.SimpleNamespace


def ints(t):
    return None if t is None else [int(x) for x in t.reshape(-1)]


class Recorder:
    """Stands in for LeapQuantState: records decode / dequantize / quantize with their slot sets and row counts."""
    HV, V, K = 4, 128, 128

    def __init__(self, log, kw):
        self.log = log
        self.kw = kw

    def decode(self, ssm, mixed, a, b, A_log, dt_bias, idx, out):
        assert mixed.is_contiguous() and b.is_contiguous()
        self.log.append(("decode", tuple(mixed.shape), tuple(a.shape), tuple(b.shape), ints(idx), tuple(out.shape)))
        out.fill_(1)

    def decode_conv(self, ssm, x, conv_state, conv_weight, conv_bias, a, b, A_log, dt_bias, idx, out):
        assert b.is_contiguous()
        self.log.append(("decode_conv", tuple(x.shape), tuple(conv_state.shape), tuple(conv_weight.shape), tuple(a.shape), ints(idx),
                         tuple(out.shape)))
        out.fill_(1)

    def dequantize(self, ssm, idx):
        self.log.append(("dequantize", ints(idx)))

    def quantize(self, ssm, idx):
        self.log.append(("quantize", ints(idx)))


class StubEngine:
    """sys.modules entries that look like the parts of vLLM the plugin imports; restore() puts the real ones back."""

    NAMES = ["vllm", "vllm.config", "vllm.forward_context", "vllm.compilation", "vllm.compilation.breakable_cudagraph",
             "vllm.model_executor", "vllm.model_executor.layers", "vllm.model_executor.layers.mamba",
             "vllm.model_executor.layers.mamba.gdn", "vllm.model_executor.layers.mamba.gdn.qwen_gdn_linear_attn",
             "vllm.model_executor.layers.mamba.mamba_utils", "vllm.model_executor.layers.mamba.ops",
             "vllm.model_executor.layers.mamba.ops.causal_conv1d", "vllm.models", "vllm.models.glm5next",
             "vllm.models.glm5next.nvidia", "vllm.models.glm5next.nvidia.kda"]

    def __init__(self, log):
        self.log = log
        self.saved = {n: sys.modules.get(n) for n in self.NAMES}
        self.ctx = NS(attn_metadata=None)
        mods = {n: types.ModuleType(n) for n in self.NAMES}
        for n, m in mods.items():
            m.__path__ = []                                       # every stub is a package: submodule imports resolve in sys.modules
            parent, _, leaf = n.rpartition(".")
            if parent:
                setattr(mods[parent], leaf, m)
        mods["vllm.forward_context"].get_forward_context = lambda: self.ctx
        mods["vllm.config"].get_current_vllm_config = lambda: NS(
            compilation_config=NS(max_cudagraph_capture_size=48), scheduler_config=NS(max_num_seqs=32))

        def eager_break_during_capture(fn):
            def wrapper(*a, **k):
                return fn(*a, **k)
            wrapper.__wrapped__ = fn
            return wrapper
        mods["vllm.compilation.breakable_cudagraph"].eager_break_during_capture = eager_break_during_capture
        mods["vllm.model_executor.layers.mamba.mamba_utils"].is_conv_state_dim_first = lambda: False

        def causal_conv1d_update(x, conv_state, weight, bias=None, activation=None, conv_state_indices=None, **kw):
            log.append(("conv_update", tuple(x.shape), tuple(conv_state.shape), tuple(weight.shape), activation,
                        ints(conv_state_indices)))
            return x + 0
        mods["vllm.model_executor.layers.mamba.ops.causal_conv1d"].causal_conv1d_update = causal_conv1d_update

        # ---- Gated DeltaNet layer module ----
        G = mods["vllm.model_executor.layers.mamba.gdn.qwen_gdn_linear_attn"]

        def engine_decode_kernel(**kw):
            log.append(("engine_decode_kernel", tuple(kw["q"].shape), ints(kw["ssm_state_indices"])))
            return torch.zeros(1, kw["q"].shape[1], 4, 128), None
        G.fused_sigmoid_gating_delta_rule_update = engine_decode_kernel

        class QwenGatedDeltaNetAttention:
            def __init__(self, **kw):
                self.__dict__.update(kw)

            def _forward_core(self, mixed_qkv, b, a, core_attn_out):
                log.append(("engine_core", tuple(mixed_qkv.shape)))
                md = self.engine_plan
                if md is not None:                                 # the engine's own decode call for the decode tokens of the step
                    q, k, v = md
                    n = q.shape[1]
                    out, _ = G.fused_sigmoid_gating_delta_rule_update(
                        A_log=self.A_log, a=a[:n], b=b[:n], dt_bias=self.dt_bias, q=q, k=k, v=v, initial_state=None,
                        inplace_final_state=True, cu_seqlens=None, ssm_state_indices=self.engine_slots,
                        use_qk_l2norm_in_kernel=True, **self.engine_kw)
                    log.append(("engine_core_got", tuple(out.shape)))
                return "engine"
        G.QwenGatedDeltaNetAttention = QwenGatedDeltaNetAttention

        # ---- Kimi Delta Attention layer module ----
        KM = mods["vllm.models.glm5next.nvidia.kda"]

        class Glm5NextLinearAttention:
            def __init__(self, **kw):
                self.__dict__.update(kw)

            def _forward(self, qkv_proj_states, g1, beta, core_attn_out):
                log.append(("engine_forward", tuple(qkv_proj_states.shape)))
        KM.Glm5NextLinearAttention = Glm5NextLinearAttention

        def causal_conv1d_fn(x, weight, bias, activation=None, conv_states=None, has_initial_state=None, cache_indices=None,
                             query_start_loc=None, metadata=None):
            log.append(("conv_fn", tuple(x.shape), tuple(weight.shape), tuple(conv_states.shape), ints(cache_indices)))
            return x + 0
        KM.causal_conv1d_fn = causal_conv1d_fn
        KM.gather_initial_states = lambda ssm, idx, has: (log.append(("gather", ints(idx), ints(has))), torch.zeros(1))[1]
        KM._cast_sigmoid = lambda t: torch.sigmoid(t.float())

        def chunk_kda_with_fused_gate(q, k, v, raw_g, beta, cu_seqlens=None, **kw):
            log.append(("chunk_kda", tuple(q.shape), tuple(raw_g.shape), tuple(beta.shape), ints(cu_seqlens), kw["lower_bound"]))
            return torch.full((1, q.shape[1], q.shape[2], q.shape[3]), 2.0), torch.zeros(1)
        KM.chunk_kda_with_fused_gate = chunk_kda_with_fused_gate
        KM.scatter_states = lambda ssm, last, idx: log.append(("scatter", ints(idx)))
        self.mods = mods
        sys.modules.update(mods)

    def restore(self):
        for n, m in self.saved.items():
            if m is None:
                sys.modules.pop(n, None)
            else:
                sys.modules[n] = m


def load_plugin(which):
    """('ours' | 'reference') -> (gdn module, glm module), freshly loaded so that each binds the current stubs."""
    if which == "ours":
        import leapquant_b200.vllm.gdn as g
        import leapquant_b200.vllm.glm as k
        return importlib.reload(g), importlib.reload(k)
    import leapquant_b200
    leapquant_b200.install_alias()
    out = []
    for name in ("gdn", "glm"):
        spec = importlib.util.spec_from_file_location(f"_reference_plugin_{name}", os.path.join(REF, "leapquant", "vllm", name + ".py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        out.append(mod)
    return tuple(out)


def gdn_layer(eng, prefix="layers.3.linear_attn"):
    H, HV, K, V, C = 2, 4, 128, 128, 2 * 2 * 128 + 4 * 128
    cls = eng.mods["vllm.model_executor.layers.mamba.gdn.qwen_gdn_linear_attn"].QwenGatedDeltaNetAttention
    return cls(prefix=prefix, num_k_heads=H * 2, tp_size=2, enable_packed_recurrent_decode=True, activation="silu",
               kv_cache=(torch.zeros(9, 3, C), torch.zeros(9, HV, V, K)), conv1d=NS(weight=torch.zeros(C, 1, 4), bias=torch.zeros(C)),
               A_log=torch.zeros(HV), dt_bias=torch.zeros(HV), engine_plan=None, engine_slots=None, engine_kw={}), C


def run_gdn_scenarios(which, fuse=False):
    log = []
    eng = StubEngine(log)
    try:
        gmod, _ = load_plugin(which)
        states = {}

        def fake_get_state(layer, ssm, **kw):
            log.append(("get_state", kw.get("H"), kw.get("nmax"), bool(kw.get("kda", False))))
            return states.setdefault(id(layer), Recorder(log, kw))
        gmod.get_state = fake_get_state
        adapter = gmod.install([48])
        if adapter is not None:
            adapter.fuse_conv = fuse                              # (the reference plugin has no fused conv: compare without it)
        layer, C = gdn_layer(eng)
        T = 6
        x, b, a, out = torch.zeros(T, C, dtype=torch.bfloat16 if fuse else torch.float32), torch.zeros(T, 4), torch.zeros(T, 4), torch.zeros(T, 4 * 128)
        I = lambda *v: torch.tensor(v, dtype=torch.int32)
        call = lambda: layer._forward_core(mixed_qkv=x, b=b, a=a, core_attn_out=out)

        log.append("-- warm-up: no metadata")
        eng.ctx.attn_metadata = None
        call()
        log.append("-- metadata of other layers only")
        eng.ctx.attn_metadata = {"layers.0.linear_attn": NS()}
        call()
        log.append("-- pure decode, 3 live rows of a padded batch")
        eng.ctx.attn_metadata = {layer.prefix: NS(spec_sequence_masks=None, num_prefills=0, num_decodes=3, num_actual_tokens=3,
                                                  non_spec_state_indices_tensor=I(4, 2, 7, 0, 0, 0), spec_state_indices_tensor=None,
                                                  prefill_state_indices=None)}
        call()
        log.append("-- mixed: 2 decode tokens rerouted, prefill slots 5 and a padding entry")
        eng.ctx.attn_metadata = {layer.prefix: NS(spec_sequence_masks=None, num_prefills=2, num_decodes=2, num_actual_tokens=6,
                                                  non_spec_state_indices_tensor=I(4, 2, 5, -1), spec_state_indices_tensor=None,
                                                  prefill_state_indices=I(5, -1))}
        layer.engine_plan = (torch.zeros(1, 2, 2, 128), torch.zeros(1, 2, 2, 128), torch.zeros(1, 2, 4, 128))
        layer.engine_slots = I(4, 2)
        call()
        log.append("-- mixed, but the engine's decode call verifies speculative tokens: not rerouted")
        layer.engine_kw = {"num_accepted_tokens": I(1, 1)}
        call()
        layer.engine_kw = {}
        log.append("-- speculative decoding: every touched slot round-trips, nothing rerouted")
        eng.ctx.attn_metadata = {layer.prefix: NS(spec_sequence_masks=torch.ones(2, dtype=torch.bool), num_prefills=0, num_decodes=1,
                                                  num_actual_tokens=5, non_spec_state_indices_tensor=I(6),
                                                  spec_state_indices_tensor=torch.tensor([[1, 2], [3, -1]], dtype=torch.int32),
                                                  prefill_state_indices=None)}
        call()
        log.append("-- no state indices at all: the engine's forward alone")
        layer.engine_plan = None
        eng.ctx.attn_metadata = {layer.prefix: NS(spec_sequence_masks=torch.ones(1, dtype=torch.bool), num_prefills=0, num_decodes=0,
                                                  num_actual_tokens=0, non_spec_state_indices_tensor=None,
                                                  spec_state_indices_tensor=None, prefill_state_indices=None)}
        call()
        log.append("-- packed decode disabled on the layer: pure decode takes the round trip")
        layer.enable_packed_recurrent_decode = False
        eng.ctx.attn_metadata = {layer.prefix: NS(spec_sequence_masks=None, num_prefills=0, num_decodes=2, num_actual_tokens=2,
                                                  non_spec_state_indices_tensor=I(3, 8), spec_state_indices_tensor=None,
                                                  prefill_state_indices=None)}
        call()
        return log
    finally:
        eng.restore()


def kda_layer(eng, prefix="layers.1.linear_attn"):
    HV, D = 4, 128
    C = 3 * HV * D
    cls = eng.mods["vllm.models.glm5next.nvidia.kda"].Glm5NextLinearAttention
    conv = lambda: NS(weight=torch.zeros(HV * D, 1, 4), bias=torch.zeros(HV * D))
    return cls(prefix=prefix, local_num_heads=HV, head_dim=D, local_projection_size=HV * D, kda_lower_bound=-5.0, kda_safe_gate=True,
               kda_prefill_backend="fla", _conv_state_dim_first=True, _merged_conv_weight=None, q_conv1d=conv(), k_conv1d=conv(),
               v_conv1d=conv(), kv_cache=(torch.zeros(9, C, 3), torch.zeros(9, HV, D, D)), A_log=torch.zeros(1, 1, HV, 1),
               dt_bias=torch.zeros(HV * D)), C


def run_kda_scenarios(which, fuse=False):
    log = []
    eng = StubEngine(log)
    try:
        _, kmod = load_plugin(which)
        states = {}

        def fake_get_state(layer, ssm, **kw):
            log.append(("get_state", kw.get("H"), kw.get("nmax"), bool(kw.get("kda", False)), kw.get("gate_lower_bound")))
            return states.setdefault(id(layer), Recorder(log, kw))
        kmod.get_state = fake_get_state
        adapter = kmod.install([16])
        if adapter is not None:
            adapter.fuse_conv = fuse
        layer, C = kda_layer(eng)
        T = 7
        x, g1, beta = torch.zeros(T, C, dtype=torch.bfloat16 if fuse else torch.float32), torch.zeros(1, T, 4, 128), torch.zeros(1, T, 4)
        out = torch.zeros(1, T, 4, 128)
        I = lambda *v: torch.tensor(v, dtype=torch.int32)
        call = lambda: layer._forward(qkv_proj_states=x, g1=g1, beta=beta, core_attn_out=out)

        log.append("-- no metadata / empty step")
        eng.ctx.attn_metadata = None
        call()
        eng.ctx.attn_metadata = {layer.prefix: NS(num_actual_tokens=0)}
        call()
        log.append("-- pure decode, 3 rows")
        eng.ctx.attn_metadata = {layer.prefix: NS(num_actual_tokens=3, spec_sequence_masks=None, num_spec_decodes=0, num_prefills=0,
                                                  non_spec_state_indices_tensor=I(4, 2, 7, 0))}
        call()
        log.append("-- mixed: 2 decode tokens first, then prefill slots 5 and 6")
        eng.ctx.attn_metadata = {layer.prefix: NS(num_actual_tokens=7, spec_sequence_masks=None, num_spec_decodes=0, num_prefills=2,
                                                  num_decode_tokens=2, non_spec_state_indices_tensor=I(4, 2, 5, 6),
                                                  has_initial_state=torch.tensor([True, True, False, True]),
                                                  non_spec_query_start_loc=I(0, 1, 2, 4, 7), prefill_state_indices=I(5, 6),
                                                  prefill_has_initial_state=torch.tensor([False, True]),
                                                  prefill_query_start_loc=I(0, 2, 5))}
        call()
        assert float(out[0, 2:7].min()) == 2.0 and float(out[0, :2].max()) == 1.0     # prefill rows from the engine, decode rows from us
        log.append("-- mixed without decode tokens")
        md = eng.ctx.attn_metadata[layer.prefix]
        md.num_decode_tokens, md.num_actual_tokens = 0, 5
        md.non_spec_state_indices_tensor, md.non_spec_query_start_loc = I(5, 6), I(0, 2, 5)
        call()
        log.append("-- speculative decoding: round trip of every touched slot around the engine's forward")
        eng.ctx.attn_metadata = {layer.prefix: NS(num_actual_tokens=4, spec_sequence_masks=torch.ones(2, dtype=torch.bool),
                                                  num_spec_decodes=2, num_prefills=0, non_spec_state_indices_tensor=I(8),
                                                  spec_state_indices_tensor=torch.tensor([[1, 2], [3, -1]], dtype=torch.int32))}
        call()
        return log
    finally:
        eng.restore()


def test_gdn_routes_and_call_sequence():
    log = run_gdn_scenarios("ours")
    sect = lambda name: log[log.index(name) + 1: next((i for i in range(log.index(name) + 1, len(log)) if isinstance(log[i], str)), len(log))]
    assert sect("-- warm-up: no metadata") == [("engine_core", (6, 1024))]
    assert sect("-- metadata of other layers only") == [("engine_core", (6, 1024))]
    dec = sect("-- pure decode, 3 live rows of a padded batch")
    assert [e[0] for e in dec] == ["conv_update", "get_state", "decode"]
    assert dec[0] == ("conv_update", (3, 1024), (9, 1024, 3), (1024, 4), "silu", [4, 2, 7])     # state handed over dim-first
    assert dec[1] == ("get_state", 2, 48, False)                                                # local key heads, recorded batch bound
    assert dec[2] == ("decode", (3, 1024), (3, 4), (3, 4), [4, 2, 7], (3, 4, 128))
    mix = sect("-- mixed: 2 decode tokens rerouted, prefill slots 5 and a padding entry")
    assert [e[0] for e in mix] == ["get_state", "dequantize", "engine_core", "get_state", "decode", "engine_core_got", "quantize"]
    assert mix[1] == ("dequantize", [5, 0]) and mix[-1] == ("quantize", [5, 0])                 # padding entry clamped to the null slot
    assert mix[4] == ("decode", (2, 1024), (2, 4), (2, 4), [4, 2], (2, 4, 128)) and mix[5] == ("engine_core_got", (1, 2, 4, 128))
    nor = sect("-- mixed, but the engine's decode call verifies speculative tokens: not rerouted")
    assert [e[0] for e in nor] == ["get_state", "dequantize", "engine_core", "engine_decode_kernel", "engine_core_got", "quantize"]
    spec = sect("-- speculative decoding: every touched slot round-trips, nothing rerouted")
    assert [e[0] for e in spec] == ["get_state", "dequantize", "engine_core", "engine_decode_kernel", "engine_core_got", "quantize"]
    assert spec[1] == ("dequantize", [6, 1, 2, 3, 0]) and spec[-1] == ("quantize", [6, 1, 2, 3, 0])
    assert [e[0] for e in sect("-- no state indices at all: the engine's forward alone")] == ["get_state", "engine_core"]
    off = sect("-- packed decode disabled on the layer: pure decode takes the round trip")
    assert [e[0] for e in off] == ["get_state", "dequantize", "engine_core", "quantize"] and off[1] == ("dequantize", [3, 8])


def test_kda_routes_and_call_sequence():
    log = run_kda_scenarios("ours")
    sect = lambda name: log[log.index(name) + 1: next((i for i in range(log.index(name) + 1, len(log)) if isinstance(log[i], str)), len(log))]
    assert sect("-- no metadata / empty step") == []
    dec = sect("-- pure decode, 3 rows")
    assert [e[0] for e in dec] == ["get_state", "conv_update", "decode"]
    assert dec[0] == ("get_state", 4, 16, True, -5.0)
    assert dec[1] == ("conv_update", (3, 1536), (9, 1536, 3), (1536, 4), "silu", [4, 2, 7])     # q | k | v conv weights merged
    assert dec[2] == ("decode", (3, 1536), (3, 4, 128), (3, 4), [4, 2, 7], (3, 4, 128))
    mix = sect("-- mixed: 2 decode tokens first, then prefill slots 5 and 6")
    assert [e[0] for e in mix] == ["get_state", "conv_fn", "decode", "dequantize", "gather", "chunk_kda", "scatter", "quantize"]
    assert mix[2] == ("decode", (2, 1536), (2, 4, 128), (2, 4), [4, 2], (2, 4, 128))
    assert mix[3] == ("dequantize", [5, 6]) and mix[4] == ("gather", [5, 6], [0, 1]) and mix[7] == ("quantize", [5, 6])
    assert mix[5] == ("chunk_kda", (1, 5, 4, 128), (1, 5, 4, 128), (1, 5, 4), [0, 2, 5], -5.0)
    nod = sect("-- mixed without decode tokens")
    assert [e[0] for e in nod] == ["get_state", "conv_fn", "dequantize", "gather", "chunk_kda", "scatter", "quantize"]
    spec = sect("-- speculative decoding: round trip of every touched slot around the engine's forward")
    assert spec == [("get_state", 4, 16, True, -5.0), ("dequantize", [8, 1, 2, 3, 0]), ("engine_forward", (7, 1536)),
                    ("quantize", [8, 1, 2, 3, 0])]


def test_pure_decode_uses_the_fused_conv_launch_by_default():
    """With the default setting a pure decode step is ONE call: conv1d update + decode, the engine's conv kernel is not called."""
    sect = lambda log, name: log[log.index(name) + 1: next((i for i in range(log.index(name) + 1, len(log)) if isinstance(log[i], str)), len(log))]
    g = sect(run_gdn_scenarios("ours", fuse=True), "-- pure decode, 3 live rows of a padded batch")
    assert [e[0] for e in g] == ["get_state", "decode_conv"]
    assert g[1] == ("decode_conv", (3, 1024), (9, 1024, 3), (1024, 4), (3, 4), [4, 2, 7], (3, 4, 128))
    k = sect(run_kda_scenarios("ours", fuse=True), "-- pure decode, 3 rows")
    assert [e[0] for e in k] == ["get_state", "decode_conv"]
    assert k[1] == ("decode_conv", (3, 1536), (9, 1536, 3), (1536, 4), (3, 4, 128), [4, 2, 7], (3, 4, 128))
    import leapquant_b200.vllm.gdn as G
    import leapquant_b200.vllm.glm as KM
    src = open(G.__file__).read() + open(KM.__file__).read()
    assert src.count("self.fuse_conv = True") == 2


@pytest.mark.skipif(not HAVE_REF, reason="reference checkout not present")
@pytest.mark.parametrize("layer_kind", ["gdn", "kda"])
def test_same_call_sequence_as_the_reference_plugin(layer_kind):
    """The reference's own plugin file, bound to this package through install_alias(), produces the same call log."""
    run = run_gdn_scenarios if layer_kind == "gdn" else run_kda_scenarios
    ours, ref = run("ours"), run("reference")
    if layer_kind == "gdn":
        # the one scenario the reference cannot serve: metadata without `prefill_state_indices` never occurs there
        assert len(ours) == len(ref)
    assert ours == ref


def test_gdn_engine_without_separate_prefill_slots_round_trips_everything():
    """An engine whose metadata lacks `prefill_state_indices` (vLLM 0.22): a mixed step round-trips every touched slot."""
    from leapquant_b200.vllm.routing import Route, plan_gdn_step
    md = NS(spec_sequence_masks=None, num_prefills=1, num_decodes=1, non_spec_state_indices_tensor=torch.tensor([3, 4], dtype=torch.int32),
            spec_state_indices_tensor=None)
    plan = plan_gdn_step(md)
    assert plan.route is Route.ROUND_TRIP and ints(plan.slots) == [3, 4]
    assert plan_gdn_step(None).route is Route.ENGINE


def test_register_installs_what_the_engine_ships():
    """register() wraps the layer constructors to record the largest decode batch and installs both adapters; a layer class
    the engine lacks is skipped without failing the other."""
    log = []
    eng = StubEngine(log)
    try:
        import leapquant_b200.vllm as P
        importlib.reload(P)
        P.register()
        G = eng.mods["vllm.model_executor.layers.mamba.gdn.qwen_gdn_linear_attn"]
        G.QwenGatedDeltaNetAttention(prefix="x")                       # constructor wrapper reads the engine config
        assert P._NMAX[0] == 48
        assert G.fused_sigmoid_gating_delta_rule_update.__name__ == "decode_kernel"
        assert hasattr(eng.mods["vllm.models.glm5next.nvidia.kda"].Glm5NextLinearAttention._forward, "__wrapped__")
        P.register()                                                   # idempotent
    finally:
        eng.restore()
        import leapquant_b200.vllm as P
        importlib.reload(P)
