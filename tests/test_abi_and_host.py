"""CPU tests of the boundary: the C-ABI library loads and exports what the header declares, argument errors come back as
codes before anything touches a GPU, and the host-side mirror of the reference API behaves like the reference's."""
import ctypes
import os
import re
import types

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    src = open(os.path.join(ROOT, "include", "leapquant_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(lq_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    from leapquant_b200 import _lib
    L = _lib.lib()
    names = header_functions()
    assert len(names) >= 10 and "lq_gdn_step" in names and "lq_flush" in names
    for n in names:
        assert hasattr(L, n), f"{n} declared in the header but not exported"
    assert sorted(_lib.EXPORTS) == [n for n in names if n in _lib.EXPORTS]
    assert L.lq_version() >= 100
    assert b"unsupported" in L.lq_strerror(-2)


def test_argument_errors_are_codes_not_crashes():
    from leapquant_b200 import _lib
    L = _lib.lib()
    good = _lib.dims(8, 4, 2, 128, 128, 16, 4, 4 * 128 * 128)
    one = ctypes.c_void_p(256)            # a non-null, 16-byte aligned dummy; never dereferenced on these paths
    assert L.lq_quantize(good, None, one, one, None, one, one, one, 1, 0, 1, None) == -1          # NULL ssm
    assert L.lq_quantize(good, one, one, one, None, one, one, one, 0, 0, 1, None) == 0            # N == 0: nothing to do
    assert L.lq_quantize(good, one, one, one, None, one, one, one, -1, 0, 1, None) == -4
    assert L.lq_quantize(good, one, one, one, None, one, one, one, 1, 1, 1, None) == -1           # KDA needs Gbuf
    for bad in (_lib.dims(8, 4, 2, 64, 128, 16, 4, 4 * 128 * 128), _lib.dims(8, 4, 2, 128, 128, 16, 3, 4 * 128 * 128),
                _lib.dims(8, 4, 2, 128, 128, 18, 4, 4 * 128 * 128), _lib.dims(8, 4, 2, 128, 128, 128, 4, 4 * 128 * 128)):
        assert L.lq_flush(bad, one, one, one, one, one, None, one, one, one, 1, 0, 1, None) == -2
    assert L.lq_flush(_lib.dims(8, 4, 3, 128, 128, 16, 4, 4 * 128 * 128), one, one, one, one, one, None, one, one, one,
                      1, 0, 1, None) == -4                                                         # HV % H != 0
    assert L.lq_flush(_lib.dims(8, 4, 2, 128, 128, 16, 4, 4 * 128 * 128 + 2), one, one, one, one, one, None, one, one, one,
                      1, 0, 1, None) == -3                                                         # slot stride alignment
    mis = ctypes.c_void_p(260)
    assert L.lq_gdn_step(good, mis, one, one, one, one, one, one, one, one, one, one, one, one, 1, 0.0, None) == -3
    # every entry point that moves the state with 128-bit accesses refuses a misaligned pointer before it launches
    assert L.lq_quantize(good, mis, one, one, None, one, one, one, 1, 0, 1, None) == -3
    assert L.lq_dequant(good, mis, one, one, one, one, None, one, one, 1, 0, None) == -3
    assert L.lq_dequant(good, one, mis, one, one, one, None, one, one, 1, 0, None) == -3
    assert L.lq_flush(good, mis, one, one, one, one, None, one, one, one, 1, 0, 1, None) == -3
    assert L.lq_flush(good, one, one, mis, one, one, None, one, one, one, 1, 0, 1, None) == -3
    assert L.lq_flush(good, one, one, one, one, one, mis, one, one, one, 1, 1, 1, None) == -3       # KDA: Gbuf
    # fused decode: the step's checks plus the flush's Q0 / iters
    dec = (good, one, one, one, one, one, one, one, one, one, one, one, one, one, 1, 0.0)
    assert L.lq_gdn_decode(*dec, None, 1, None, 0, None) == -1                                       # NULL Q0
    assert L.lq_gdn_decode(*dec, one, -1, None, 0, None) == -4                                       # negative iters
    assert L.lq_gdn_decode(good, mis, *dec[2:], one, 1, None, 0, None) == -3                         # misaligned state
    assert L.lq_gdn_decode(*dec[:14], 0, 0.0, one, 1, None, 0, None) == 0                            # N == 0
    assert L.lq_gdn_decode(*dec, one, 1, one, 16, None) == -4                                        # mailbox scratch too small
    assert L.lq_decode_work_bytes(8, 4) == 4 * (16 + 4 * 1024)
    assert L.lq_kda_decode(good, one, one, one, one, one, None, one, one, one, one, one, one, one, one, 1, 0.0, 0.0, one, 1,
                           None, 0, None) == -1                                                      # KDA needs Gbuf
    assert L.lq_set_option(b"pdl", 1) == 0 and L.lq_set_option(b"no_such_option", 1) == -2
    assert L.lq_lowrank(one, one, one, one, 1, 64, 128, 4, 3, None) == -2
    assert L.lq_lowrank(one, one, one, one, 0, 128, 128, 4, 3, None) == 0


def test_host_tensors_are_refused():
    from leapquant_b200 import _lib
    from leapquant_b200.kernels import make_quantize
    from leapquant_b200.state import LeapQuantState
    with pytest.raises(RuntimeError):
        LeapQuantState(torch.zeros(2, 2, 128, 128), 2)
    q = make_quantize(2, 2, 128, 128, 16, 2 * 128 * 128)
    t = torch.zeros(2, 2, 128, 128)
    with pytest.raises(_lib.LeapQuantError):
        q(t, t, t, t, t, t, t, t, t, torch.zeros(1, dtype=torch.int32))


def test_unsupported_shapes_raise_not_implemented():
    from leapquant_b200 import kernels as KN
    with pytest.raises(NotImplementedError):
        KN.make_gdn_step(8, 4, 2, 64, 128, 16, 4 * 64 * 128)
    with pytest.raises(NotImplementedError):
        KN.make_flush(8, 4, 64, 64, 16, 4 * 64 * 64)
    # the reference's tuning keywords are accepted
    KN.make_gdn_step(8, 4, 2, 128, 128, 16, 4 * 128 * 128, R=4, SMS=148, NSTAGE=6, NCG=3, NNW=2, MAXIT=256)
    KN.make_kda_step(8, 4, 2, 128, 128, 16, 4 * 128 * 128, R=4, SMS=148, NSTAGE=6, NSTAGEQ=4, NCG=2, NNW=3, GLB=-5.0)
    KN.make_flush(8, 4, 128, 128, 16, 4 * 128 * 128, R=4, ITERS=1, SMS=148, NCG=3, KDA=True, NMAX=64)
    assert KN.QMAX == 127.0 and KN.EPS == 1e-12 and KN.SOFTPLUS_THRESHOLD == 20.0 and (128, 128) in KN.STEP_CFG


def test_api_surface_matches_reference_names():
    import leapquant_b200
    from leapquant_b200 import kernels as KN, state as ST
    for n in ("make_gdn_step", "make_kda_step", "make_flush", "make_dequant", "make_quantize", "make_lowrank",
              "lowrank_factor", "F32", "BF16", "I32", "I8"):
        assert hasattr(KN, n), n
    for n in ("LeapQuantState", "state_views", "get_state", "WINDOW", "RANK", "_ident"):
        assert hasattr(ST, n), n
    assert ST.WINDOW == 16 and ST.RANK == 4
    pkg = leapquant_b200.install_alias("leapquant_alias_for_test")
    import importlib
    assert importlib.import_module("leapquant_alias_for_test.state") is ST
    import leapquant_b200.vllm as PV
    assert callable(PV.register)


def test_get_state_caching_and_prefix_cache_guard(monkeypatch):
    """get_state: same tensor -> same object; a re-allocated cache bumps the generation and drops the old states;
    prefix caching of the recurrent state is refused (reference leapquant/state.py:172-189)."""
    from leapquant_b200 import state as ST
    made = []

    class Fake:
        def __init__(self, ssm, **kw):
            self.key = ST._ident(ssm)
            self.kw = kw
            made.append(self)

    monkeypatch.setattr(ST, "LeapQuantState", Fake)
    monkeypatch.setattr(torch.cuda, "empty_cache", lambda: None)
    ST._STATES.clear()
    ST._GEN[0] = 0
    a, b = types.SimpleNamespace(), types.SimpleNamespace()
    t1 = torch.zeros(2, 2, 4, 4)
    s1 = ST.get_state(a, t1, H=2)
    assert ST.get_state(a, t1, H=2) is s1 and len(made) == 1
    assert ST.get_state(b, t1, H=2) is s1                         # two layers sharing one state tensor share the state
    assert ST.get_state(a, t1[:1], H=2) is not s1                 # a different view is a different state, cache dropped
    assert ST._GEN[0] == 1 and len(ST._STATES) == 1
    guarded = types.SimpleNamespace(cache_config=types.SimpleNamespace(mamba_cache_mode="all"))
    with pytest.raises(RuntimeError, match="prefix caching"):
        ST.get_state(guarded, torch.zeros(3, 2, 4, 4), H=2)
    ST._STATES.clear()


def test_sharding_partitions():
    from leapquant_b200.sharding import shard_heads, shard_rows, slice_mixed_heads
    for n, w in ((1024, 8), (10, 4), (3, 8), (0, 2)):
        spans = [shard_rows(n, w, r) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(spans[i][1] == spans[i + 1][0] for i in range(w - 1))
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= 1
    assert shard_heads(16, 32, 8, 3) == ((6, 8), (12, 16))
    with pytest.raises(ValueError):
        shard_heads(16, 32, 3, 0)
    H, HV, K, V = 4, 8, 2, 3
    mixed = torch.arange(5 * (2 * H * K + HV * V)).view(5, -1)
    parts = [slice_mixed_heads(mixed, H, HV, K, V, 2, r) for r in range(2)]
    assert parts[0].shape == (5, 2 * 2 * K + 4 * V)
    assert torch.equal(parts[1][:, :2 * K], mixed[:, 2 * K:4 * K])
    assert torch.equal(parts[1][:, -4 * V:], mixed[:, -4 * V:])
