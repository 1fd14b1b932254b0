"""CPU oracle for LeapQuant's quantized-state decode path.  TEST INFRASTRUCTURE ONLY.

This module is a restatement, in plain fp32 PyTorch on CPU tensors, of the arithmetic of the reference's
TileLang CUDA kernels.  The reference has no CPU or PyTorch implementation of the decode step, the flush or the
GDN quantize/dequant (all are CUDA kernels generated at run time), and it ships no tests, golden vectors or
fixtures, so:

  * parity of the decode-step and flush restatements is UNPINNED by reference outputs (their kernels were not run: the
    generated code of the step kernel did not build here, and both spin on flags without a bound);
  * the packed layout (`state_views`) and the KDA torch round trip (`kda_rebuild`, `kda_checkpoint`) ARE pinned
    against the reference's own Python code (fixtures under tests/golden/, produced by tests/golden/make_golden.py);
  * the GDN quantize, the dequantize and the low-rank factorisation ARE pinned against outputs of the reference's own
    TileLang kernels, run once on a B200 (fixtures under tests/golden/ref_kernels/, produced by
    tests/golden/make_ref_kernel_golden.py; tests/test_ref_kernel_golden.py).

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / `--impl reference` leg may import this module.
The product (leapquant_b200) never imports it and has no CPU fallback.

Conventions (leapquant/state.py:1-6,29-40): one (slot, value head) of the fp32 state tensor [NS, HV, V, K] holds, in
order, the INT8 codes [V][K], the column scales Sk f32[K], the row scales Sv f32[V] and the fp16 Compensator-Token
factors [R][K+V] = U^T | Q^T.  The dequantised checkpoint is  S0[v,c] = q8[v,c]/127 * Sk[c] * Sv[v] + sum_r Q[r][v] U[r][c].
The live state is  p * S0 (+ per-channel decay for KDA)  +  sum_{j<h} w_j u_j (x) k_j  over the window buffer.

Where the reference keeps a transient tile in reduced precision only because of its tensor-core operand format (the
fp16 B / E tile of the flush, the bf16 hi+lo split of the rebuild operands, the fp16 hi+lo split of the step's
matvec operand, the fp16 `pc * U^T` of the KDA flush), this oracle computes in fp32 and says so at the spot.  Every
rounding that defines a STORED value (bf16 window appends, bf16 beta, fp16 factors, fp16 per-entry decay factors,
INT8 codes, the fp16 operand tiles P / Q of the subspace iteration) is mirrored.
"""
import math

import torch

QMAX = 127.0
EPS = 1e-12
SOFTPLUS_THRESHOLD = 20.0
PNMIN = 1e-20
MAGIC = 12582912.0          # 1.5 * 2**23: adding it rounds an fp32 to the nearest integer (ties to even)


# --------------------------------------------------------------------------------------------------------------
# packed layout
# --------------------------------------------------------------------------------------------------------------
def _view(ssm, dtype, shape, stride, offset):
    return torch.empty(0, dtype=dtype, device=ssm.device).set_(ssm.untyped_storage()).as_strided(shape, stride, offset)


def state_views(ssm, R):
    """Aliasing views of the 8-bit checkpoint inside the fp32 state tensor [NS, HV, V, K] (leapquant/state.py:29-40).

    Offsets in units of each view's element type: codes at byte 0, scales at float V*K/4, factors at half
    2*(V*K/4 + K + V)."""
    NS, HV, V, K = ssm.shape
    SS = ssm.stride(0)
    off = ssm.storage_offset()
    sc = off + V * K // 4
    return dict(
        Sq=_view(ssm, torch.int8, (NS, HV, V, K), (4 * SS, 4 * V * K, K, 1), 4 * off),
        q32=_view(ssm, torch.int32, (NS, HV, V, K // 4), (SS, V * K, K // 4, 1), off),
        sq16=_view(ssm, torch.int16, (NS, HV, V, K // 2), (2 * SS, 2 * V * K, K // 2, 1), 2 * off),
        Sk=_view(ssm, torch.float32, (NS, HV, K), (SS, V * K, 1), sc),
        Sv=_view(ssm, torch.float32, (NS, HV, V), (SS, V * K, 1), sc + K),
        skv=_view(ssm, torch.float32, (NS, HV, K + V), (SS, V * K, 1), sc),
        uq=_view(ssm, torch.float16, (NS, HV, R, K + V), (2 * SS, 2 * V * K, K + V, 1), 2 * (sc + K + V)))


def checkpoint_bytes(K, V, R):
    """Bytes of one head's checkpoint inside its 4*V*K-byte slot (capacity assert: leapquant/state.py:55)."""
    return V * K + 4 * (K + V) + 2 * R * (K + V)


class Buffers:
    """The window buffers of one layer with the reference's initial values (leapquant/state.py:61-70)."""

    def __init__(self, NS, HV, K, V, L, R, kda=False, device="cpu"):
        KA = K if kda else 1
        self.kda, self.NS, self.HV, self.K, self.V, self.L, self.R = kda, NS, HV, K, V, L, R
        self.Kbuf = torch.zeros(NS, HV, L, K, dtype=torch.bfloat16, device=device)
        self.Ubuf = torch.zeros(NS, HV, L, V, dtype=torch.bfloat16, device=device)
        self.Wbuf = torch.zeros(NS, HV, L, device=device)
        self.Pbuf = torch.zeros(NS, HV, KA, device=device) if kda else torch.ones(NS, HV, 1, device=device)
        self.Gbuf = (torch.ones(NS, HV, L, KA, dtype=torch.float16, device=device) if kda
                     else torch.zeros(NS, HV, L, 1, device=device))
        self.hcnt = torch.zeros(NS, HV, dtype=torch.int32, device=device)
        self.Q0 = make_q0(V, R).to(device)

    def clone(self):
        o = object.__new__(Buffers)
        for k, v in self.__dict__.items():
            setattr(o, k, v.clone() if torch.is_tensor(v) else v)
        return o


def make_q0(V, R):
    """Fixed start of the subspace iteration: randn(V, R) from a CPU generator seeded 0 (leapquant/state.py:70)."""
    return torch.randn(V, R, generator=torch.Generator().manual_seed(0))


# --------------------------------------------------------------------------------------------------------------
# small helpers
# --------------------------------------------------------------------------------------------------------------
def _bf16(x):
    return x.to(torch.bfloat16).to(torch.float32)


def _f16(x):
    return x.to(torch.float16).to(torch.float32)


def _softplus(x):
    """log(1 + exp(x)), linear above the threshold (leapquant/kernels.py:142)."""
    return torch.where(x <= SOFTPLUS_THRESHOLD, torch.log(1.0 + torch.exp(torch.clamp(x, max=SOFTPLUS_THRESHOLD))), x)


def _qkv(mixed, rows, H, HV, K, V, scale):
    """q, k, v of the selected rows, l2-normalised as in leapquant/kernels.py:184-186,237-247,277.

    Returns qn, kn [n, HV, K] (the key head's vectors repeated over its GQA value heads), v [n, HV, V], kq [n, HV]."""
    GQA = HV // H
    m = mixed[rows].to(torch.float32)
    q = m[:, :H * K].reshape(-1, H, K)
    k = m[:, H * K:2 * H * K].reshape(-1, H, K)
    v = m[:, 2 * H * K:].reshape(-1, HV, V)
    nq = (q * q).sum(-1)
    nk = (k * k).sum(-1)
    nkq = (k * q).sum(-1)
    inq = torch.rsqrt(nq + 1e-6) * scale
    ink = torch.rsqrt(nk + 1e-6)
    qn = (q * inq[..., None]).repeat_interleave(GQA, dim=1)
    kn = (k * ink[..., None]).repeat_interleave(GQA, dim=1)
    kq = (nkq * inq * ink).repeat_interleave(GQA, dim=1)
    return qn, kn, v, kq


def _dequant_codes(q8, Sk, Sv):
    """q8 / 127 * Sk[c] * Sv[v], evaluation order of leapquant/kernels.py:2107."""
    return (q8.to(torch.float32) / QMAX) * Sk[..., None, :] * Sv[..., :, None]


# --------------------------------------------------------------------------------------------------------------
# a1: GDN decode step   (leapquant/kernels.py:27-692, K = V = 128 / HP == 1 branches)
# --------------------------------------------------------------------------------------------------------------
def gdn_step(Sq, Sk, Sv, Kbuf, Ubuf, Wbuf, Pbuf, hcnt, mixed, a, b, A_log, dt_bias, UQ, idx, o, H, scale=None):
    """One decode token per row n of `mixed`; mutates the window buffers and writes o[n] (bf16).

    Sq int8 [NS,HV,V,K], Sk/Sv f32, UQ f16 [NS,HV,R,K+V]: the `state_views` of the state tensor.
    mixed bf16 [N, 2HK + HV*V]; a [N,HV(,1)], b [N,HV] bf16; A_log [HV], dt_bias [HV(,1)] f32; idx int [N].
    Rows with idx <= 0 write zeros to o and touch nothing else (leapquant/kernels.py:374-378)."""
    NS, HV, V, K = Sq.shape
    L = Kbuf.shape[2]
    scale = K ** -0.5 if scale is None else scale
    idx = idx.to(torch.int64)
    rows = torch.nonzero(idx > 0).flatten()
    dead = torch.nonzero(idx <= 0).flatten()
    if dead.numel():
        o[dead] = 0
    if rows.numel() == 0:
        return
    sl = idx[rows]
    qn, kn, v, kq = _qkv(mixed, rows, H, HV, K, V, scale)
    # gates (leapquant/kernels.py:141-144)
    xg = a.reshape(a.shape[0], HV)[rows].to(torch.float32) + dt_bias.reshape(HV).to(torch.float32)
    alpha = torch.exp(-torch.exp(A_log.to(torch.float32).reshape(HV)) * _softplus(xg))
    beta = _bf16(torch.sigmoid(b[rows].to(torch.float32)))
    h = hcnt[sl].to(torch.int64)                                   # [n, HV]
    assert int(h.max()) < L, "decode step on a full window: the flush has not run"
    live = torch.arange(L)[None, None, :] < h[..., None]           # [n, HV, L]
    # window weights decay, written back for j < h only (leapquant/kernels.py:270-274)
    W = Wbuf[sl]
    Wn = torch.where(live, W * alpha[..., None], W)
    pn = Pbuf[sl][..., 0] * alpha                                  # leapquant/kernels.py:278
    # checkpoint matvec (leapquant/kernels.py:255-267,390-404,537-538).  The reference splits the operand
    # k_hat*Sk/127 into fp16 hi + lo for its tensor-core stream (fp32-level accuracy); here it is plain fp32.
    skq = Sk[sl] * (1.0 / QMAX)
    q8 = Sq[sl].to(torch.float32)                                  # [n, HV, V, K]
    svv = Sv[sl]
    mq = torch.einsum("nhvc,nhc->nhv", q8, kn * skq) * svv
    yq = torch.einsum("nhvc,nhc->nhv", q8, qn * skq) * svv
    # window dots over the stored bf16 keys and factor dots (leapquant/kernels.py:412-482); entries j >= h carry weight 0
    Kb = Kbuf[sl].to(torch.float32)
    Ub = Ubuf[sl].to(torch.float32)
    wl = torch.where(live, Wn, torch.zeros_like(Wn))
    dk = torch.einsum("nhjc,nhc->nhj", Kb, kn)
    dq = torch.einsum("nhjc,nhc->nhj", Kb, qn)
    uq = UQ[sl].to(torch.float32)
    Ut, Qt = uq[..., :K], uq[..., K:]
    dUk = torch.einsum("nhrc,nhc->nhr", Ut, kn)
    dUq = torch.einsum("nhrc,nhc->nhr", Ut, qn)
    # contribution, delta-rule correction, output (leapquant/kernels.py:539-574)
    ck = torch.einsum("nhjv,nhj->nhv", Ub, wl * dk)
    cq = torch.einsum("nhjv,nhj->nhv", Ub, wl * dq)
    rk = torch.einsum("nhrv,nhr->nhv", Qt, dUk)
    rq = torch.einsum("nhrv,nhr->nhv", Qt, dUq)
    u = beta[..., None] * (v - (pn[..., None] * (mq + rk) + ck))
    y = pn[..., None] * (yq + rq) + cq + kq[..., None] * u
    o[rows] = y.to(o.dtype)
    # appends (leapquant/kernels.py:575-585)
    n_i = torch.arange(sl.numel())[:, None].expand(-1, HV)
    hv_i = torch.arange(HV)[None, :].expand(sl.numel(), -1)
    s_i = sl[:, None].expand(-1, HV)
    Wn[n_i, hv_i, h] = 1.0
    Wbuf[sl] = Wn
    Ubuf[s_i, hv_i, h] = u.to(torch.bfloat16)
    Kbuf[s_i, hv_i, h] = kn.to(torch.bfloat16)
    Pbuf[sl] = pn[..., None]
    hcnt[sl] = (h + 1).to(hcnt.dtype)


# --------------------------------------------------------------------------------------------------------------
# a2: KDA decode step   (leapquant/kernels.py:694-1075)
# --------------------------------------------------------------------------------------------------------------
def kda_gate(xg, ea, pb, glb):
    """Per-channel log-decay g, cumulative log-gate gn and the step factor en = exp(g) (leapquant/kernels.py:708-712).

    glb != 0: bounded gate g = glb * sigmoid(ea * xg);  glb == 0: g = -ea * softplus(xg).
    en is evaluated from g directly, never as exp(gn - pb)."""
    if glb != 0.0:
        spg = 1.0 / (1.0 + torch.exp(-ea * xg))
        g = glb * spg
    else:
        g = -ea * _softplus(xg)
    return pb + g, torch.exp(g)


def kda_decay(E, h, en=None):
    """D_j = (en *) prod_{j < i < h} e_i for j < h (leapquant/kernels.py:966-979 step, 1456-1463 flush).

    E: [..., L, K] per-entry step factors (fp16 values as fp32), h: [...] live entries.  Entries j >= h get 0."""
    L = E.shape[-2]
    live = (torch.arange(L)[:, None] < h[..., None, None])
    E1 = torch.where(live, E, torch.ones_like(E))
    D = torch.ones_like(E)
    cur = torch.ones_like(E[..., 0, :]) if en is None else en.clone()
    for j in range(L - 1, -1, -1):                                 # backward running product, same order as the kernels
        D[..., j, :] = cur
        cur = cur * E1[..., j, :]
    return torch.where(live, D, torch.zeros_like(D))


def kda_step(Sq, Sk, Sv, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, mixed, a, b, A_log, dt_bias, UQ, idx, o, H,
             scale=None, glb=0.0):
    """KDA decode step: as gdn_step with a gate per key channel.  a bf16 [N,HV,K]; dt_bias f32 [HV,K];
    Pbuf f32 [NS,HV,K] holds the cumulative LOG gate; Gbuf f16 [NS,HV,L,K] each entry's step factor."""
    NS, HV, V, K = Sq.shape
    L = Kbuf.shape[2]
    scale = K ** -0.5 if scale is None else scale
    idx = idx.to(torch.int64)
    rows = torch.nonzero(idx > 0).flatten()
    dead = torch.nonzero(idx <= 0).flatten()
    if dead.numel():
        o[dead] = 0
    if rows.numel() == 0:
        return
    sl = idx[rows]
    qn, kn, v, kq = _qkv(mixed, rows, H, HV, K, V, scale)
    xg = a.reshape(a.shape[0], HV, K)[rows].to(torch.float32) + dt_bias.reshape(HV, K).to(torch.float32)
    ea = torch.exp(A_log.to(torch.float32).reshape(HV))[None, :, None]
    gn, en = kda_gate(xg, ea, Pbuf[sl], float(glb))                # leapquant/kernels.py:887-896
    pc = torch.exp(gn)
    beta = _bf16(torch.sigmoid(b[rows].to(torch.float32)))
    h = hcnt[sl].to(torch.int64)
    assert int(h.max()) < L, "decode step on a full window: the flush has not run"
    live = torch.arange(L)[None, None, :] < h[..., None]
    # checkpoint operand carries pc (leapquant/kernels.py:900-901); fp32 here (fp16 hi + lo in the reference)
    skq = Sk[sl] * (1.0 / QMAX) * pc
    q8 = Sq[sl].to(torch.float32)
    svv = Sv[sl]
    mq = torch.einsum("nhvc,nhc->nhv", q8, kn * skq) * svv
    yq = torch.einsum("nhvc,nhc->nhv", q8, qn * skq) * svv
    # window keys decayed by D_j and rounded to bf16 before the dots (leapquant/kernels.py:966-979)
    D = kda_decay(Gbuf[sl].to(torch.float32), h, en)
    Kd = _bf16(Kbuf[sl].to(torch.float32) * D)
    Ub = Ubuf[sl].to(torch.float32)
    wl = torch.where(live, Wbuf[sl], torch.zeros_like(Wbuf[sl]))
    dk = torch.einsum("nhjc,nhc->nhj", Kd, kn) * wl                # w_j folded into the dots (leapquant/kernels.py:1031-1035)
    dq = torch.einsum("nhjc,nhc->nhj", Kd, qn) * wl
    uq = UQ[sl].to(torch.float32)
    Ut, Qt = uq[..., :K] * pc[..., None, :], uq[..., K:]           # factor dots carry pc in fp32 (leapquant/kernels.py:1040)
    dUk = torch.einsum("nhrc,nhc->nhr", Ut, kn)
    dUq = torch.einsum("nhrc,nhc->nhr", Ut, qn)
    ck = torch.einsum("nhjv,nhj->nhv", Ub, dk)
    cq = torch.einsum("nhjv,nhj->nhv", Ub, dq)
    rk = torch.einsum("nhrv,nhr->nhv", Qt, dUk)
    rq = torch.einsum("nhrv,nhr->nhv", Qt, dUq)
    u = beta[..., None] * (v - (mq + rk + ck))                     # leapquant/kernels.py:1065-1066
    y = yq + rq + cq + kq[..., None] * u
    o[rows] = y.to(o.dtype)
    n_i = torch.arange(sl.numel())[:, None].expand(-1, HV)
    hv_i = torch.arange(HV)[None, :].expand(sl.numel(), -1)
    s_i = sl[:, None].expand(-1, HV)
    Pbuf[sl] = gn                                                  # leapquant/kernels.py:895-896
    Gbuf[s_i, hv_i, h] = en.to(Gbuf.dtype)
    Ubuf[s_i, hv_i, h] = u.to(torch.bfloat16)                      # leapquant/kernels.py:1067-1072
    Kbuf[s_i, hv_i, h] = kn.to(torch.bfloat16)
    Wbuf[s_i, hv_i, h] = 1.0
    hcnt[sl] = (h + 1).to(hcnt.dtype)


# --------------------------------------------------------------------------------------------------------------
# a3: window flush   (leapquant/kernels.py:1077-2033, 128 x 128 branches)
# --------------------------------------------------------------------------------------------------------------
def cholesky_qr(Q, drop):
    """One CholeskyQR pass on the columns of Q [..., V, R] in fp32 with the reference's pivot handling.

    drop=False (R <= 4, leapquant/kernels.py:1816-1829): a dependent column's pivot is floored at 1e-6 * g_jj.
    drop=True  (R == 8, leapquant/kernels.py:1760-1774): a dependent column is zeroed."""
    R = Q.shape[-1]
    G = torch.einsum("...vr,...vc->...rc", Q, Q)
    lead = Q.shape[:-2]
    Lm = torch.zeros(*lead, R, R)                                  # off-diagonal entries of the Cholesky factor
    inv = torch.zeros(*lead, R)                                    # reciprocals of its diagonal
    for j in range(R):
        for k in range(j):
            acc = G[..., j, k].clone()
            for m in range(k):
                acc = acc - Lm[..., j, m] * Lm[..., k, m]
            Lm[..., j, k] = acc * inv[..., k]
        d = G[..., j, j].clone()
        for m in range(j):
            d = d - Lm[..., j, m] * Lm[..., j, m]
        if drop:
            ok = d > 1e-6 * G[..., j, j] + 1e-30
            inv[..., j] = torch.where(ok, torch.rsqrt(torch.clamp(d, min=1e-30)), torch.zeros_like(d))
        else:
            inv[..., j] = torch.rsqrt(torch.clamp(torch.maximum(d, 1e-6 * G[..., j, j]), min=1e-30))
    out = Q.clone()
    for j in range(R):                                             # forward substitution on every row
        acc = out[..., j].clone()
        for m in range(j):
            acc = acc - out[..., m] * Lm[..., j, m][..., None]
        out[..., j] = acc * inv[..., j][..., None]
    return out


def quant_stage(E, rsk):
    """Row-wise INT8 stage of the flush (leapquant/kernels.py:1974-2013): x = E * rsk[c]; Sv[v] = max(max_c |x|, EPS);
    code = RNE(x * (127 * rcp(Sv))) by the add-1.5*2^23 trick with the product fused into the add.  No clamp."""
    x = E * rsk[..., None, :]
    Sv = torch.clamp(x.abs().amax(-1), min=EPS)
    rm = QMAX * (1.0 / Sv)
    t = (x.to(torch.float64) * rm[..., :, None].to(torch.float64) + MAGIC).to(torch.float32)      # fma(x, rm, MAGIC)
    code = (t - MAGIC).to(torch.int8)
    return Sv, code


def column_scales(E):
    """Sk[c] = max(sqrt(mean_v |E[v,c]|), EPS) (leapquant/kernels.py:1955-1957) and the reciprocal the INT8 stage
    multiplies by.  The reference takes min(rsqrt(mean), 1/EPS) with the hardware's approximate rsqrt (2 ulp); here the
    reciprocal is the correctly rounded 1 / Sk of the STORED scale, so that codes are a function of stored values only."""
    V = E.shape[-2]
    msum = E.abs().sum(-2) * (1.0 / V)
    sk = torch.clamp(torch.sqrt(msum), min=EPS)
    return sk, 1.0 / sk


def flush_rebuild(q8, Sk, Sv, Kb, Ub, w, P, G, uq_old, kda, round_b=True):
    """B (the window-rebuilt state without the old rank-R part), the scaled old factors and the scalar decay p.

    GDN (leapquant/kernels.py:1471,1483,1512-1563): p = max(Pbuf, 1e-20); B = q8 * (Sv p / 127) * Sk + sum_j (w_j u_j) k_j^T.
    KDA (leapquant/kernels.py:1448-1468,1519): pc = exp(Pbuf); keys pre-decayed by w_j D_j (D_{L-1} = 1, D_j = D_{j+1} e_{j+1});
    old U^T scaled by pc; B = q8 * (Sv / 127) * (Sk pc) + sum_j u_j (w_j D_j k_j)^T; p = 1.
    The reference holds w_j u_j (GDN) / the decayed keys (KDA) as bf16 hi + lo (16 mantissa bits): fp32 here (the split
    keeps 16 mantissa bits, below every tolerance of the parity tests).  pc * U^T and B are rounded to fp16 like the
    reference's operand tiles (leapquant/kernels.py:1466,1483): B is the A operand of every later tensor-core product.
    round_b=False returns B before that rounding (the tests use it to find the elements that sit on a rounding midpoint)."""
    K = q8.shape[-1]
    Ut, Qt = uq_old[..., :K].to(torch.float32), uq_old[..., K:].to(torch.float32)
    x = q8.to(torch.float32)
    if kda:
        L = Kb.shape[-2]
        pc = torch.exp(P)                                          # [D, K]
        h = torch.full(P.shape[:-1], L, dtype=torch.int64)
        Dj = kda_decay(G.to(torch.float32), h)                     # en = 1: D_{L-1} = 1
        kd = Kb.to(torch.float32) * (w[..., None] * Dj)
        B = x * (Sv * (1.0 / QMAX))[..., :, None] * (Sk * pc)[..., None, :]
        B = B + torch.einsum("djv,djc->dvc", Ub.to(torch.float32), kd)
        return (_f16(B) if round_b else B), _f16(Ut * pc[..., None, :]), Qt, torch.ones(P.shape[:-1])
    p = torch.clamp(P[..., 0], min=PNMIN)
    B = x * (Sv * (p / QMAX)[..., None])[..., :, None] * Sk[..., None, :]
    B = B + torch.einsum("djv,djc->dvc", w[..., None] * Ub.to(torch.float32), Kb.to(torch.float32))
    return (_f16(B) if round_b else B), Ut, Qt, p


def flush_factors(B, Ut_old, Qt_old, p, Q0, iters=1):
    """Subspace iteration of the flush on T = B + p Q_old U_old^T from the fixed start Q0, CholeskyQR twice per round
    (leapquant/kernels.py:1573-1842).  Returns the new fp16-valued factors U^T [D,R,K], Q^T [D,R,V] as fp32."""
    R = Q0.shape[1]
    Q = _f16(Q0)[None].expand(B.shape[0], -1, -1)                  # leapquant/kernels.py:1573-1577
    pp = p[:, None, None]

    def TtQ(Qm):   # P = B^T Q + p U_old (Q_old^T Q), rounded to the fp16 operand tile (leapquant/kernels.py:1581-1658)
        M = torch.einsum("drv,dvs->drs", Qt_old, Qm)
        return _f16(torch.einsum("dvc,dvr->dcr", B, Qm) + pp * torch.einsum("drc,drs->dcs", Ut_old, M))

    P = TtQ(Q)
    for _ in range(iters):
        M2 = torch.einsum("drc,dcs->drs", Ut_old, P)               # leapquant/kernels.py:1661-1718
        Qf = torch.einsum("dvc,dcr->dvr", B, P) + pp * torch.einsum("drv,drs->dvs", Qt_old, M2)
        Qf = cholesky_qr(cholesky_qr(Qf, R > 4), R > 4)            # leapquant/kernels.py:1741-1835
        Q = _f16(Qf)
        P = TtQ(Q)
    return P.transpose(-1, -2).contiguous(), Q.transpose(-1, -2).contiguous()


def flush_residual(B, Ut_old, Qt_old, p, Ut_new, Qt_new):
    """E = B + p Q_old U_old^T - Q U^T (leapquant/kernels.py:1880-1928; fp32 here, fp16 tile in the reference)."""
    return (B + p[:, None, None] * torch.einsum("drv,drc->dvc", Qt_old, Ut_old)
            - torch.einsum("drv,drc->dvc", Qt_new, Ut_new))


def flush(Sq, Sk, Sv, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, UQ, Q0, idx, kda=False, iters=1):
    """Flush every (slot, head) of the rows idx whose window is full (slot > 0 and hcnt == L, leapquant/kernels.py:1200)."""
    NS, HV, V, K = Sq.shape
    L = Kbuf.shape[2]
    idx = idx.to(torch.int64)
    sl_all = idx[idx > 0]
    if sl_all.numel() == 0:
        return 0
    due = hcnt[sl_all].to(torch.int64) == L                        # [n, HV]
    nn, hh = torch.nonzero(due, as_tuple=True)
    if nn.numel() == 0:
        return 0
    ss = sl_all[nn]
    uq_old = UQ[ss, hh]
    B, Ut_o, Qt_o, p = flush_rebuild(Sq[ss, hh], Sk[ss, hh], Sv[ss, hh], Kbuf[ss, hh], Ubuf[ss, hh], Wbuf[ss, hh],
                                     Pbuf[ss, hh], Gbuf[ss, hh] if kda else None, uq_old, kda)
    Ut_n, Qt_n = flush_factors(B, Ut_o, Qt_o, p, Q0, iters)
    E = flush_residual(B, Ut_o, Qt_o, p, Ut_n, Qt_n)
    sk, rsk = column_scales(E)
    sv, code = quant_stage(E, rsk)
    UQ[ss, hh] = torch.cat([Ut_n, Qt_n], -1).to(torch.float16)     # leapquant/kernels.py:1837-1842
    Sk[ss, hh] = sk
    Sv[ss, hh] = sv
    Sq[ss, hh] = code
    Wbuf[ss, hh] = 0.0                                             # resets (leapquant/kernels.py:2014-2031)
    if kda:
        Pbuf[ss, hh] = 0.0
        Gbuf[ss, hh] = 1.0
    else:
        Pbuf[ss, hh] = 1.0
    hcnt[ss, hh] = 0
    return int(nn.numel())


# --------------------------------------------------------------------------------------------------------------
# a4 / a5 / a6: standalone quantize, dequant, low-rank factorisation
# --------------------------------------------------------------------------------------------------------------
def mgs(X):
    """Modified Gram-Schmidt on the columns of X [..., M, R] in fp32 (leapquant/kernels.py:2170-2183)."""
    X = X.clone()
    R = X.shape[-1]
    for j in range(R):
        for c in range(j):
            s = (X[..., c] * X[..., j]).sum(-1, keepdim=True)
            X[..., j] = X[..., j] - s * X[..., c]
        nrm = torch.rsqrt(torch.clamp((X[..., j] * X[..., j]).sum(-1, keepdim=True), min=1e-30))
        X[..., j] = X[..., j] * nrm
    return X


def quantize_heads(S, Q0, iters=1):
    """8-bit checkpoint of fp32 states S [D, V, K] (leapquant/kernels.py:2161-2229): `iters` rounds of
    P = S^T Q -> MGS -> Q = S P -> MGS; U = fp16(S^T Q), Q = fp16(Q); E = S - Q U^T;
    Sk = max(sqrt(mean_v |E|), EPS); Sv = max(max_c |E / Sk|, EPS); code = clamp(nearbyint(E / (Sk Sv) * 127))."""
    Q = Q0[None].expand(S.shape[0], -1, -1).clone()
    for _ in range(iters):
        P = mgs(torch.einsum("dvc,dvr->dcr", S, Q))
        Q = mgs(torch.einsum("dvc,dcr->dvr", S, P))
    U = _f16(torch.einsum("dvc,dvr->dcr", S, Q))                   # [D, K, R]
    Q = _f16(Q)
    E = S.clone()
    for r in range(Q0.shape[1]):                                   # acc -= Q[v,r] U[c,r], one factor at a time (fused multiply-add)
        E = (E.to(torch.float64) - Q[:, :, None, r].to(torch.float64) * U[:, None, :, r].to(torch.float64)).to(torch.float32)
    sk, sv, code = quantize_stage(E)
    return code, sk, sv, torch.cat([U.transpose(-1, -2), Q.transpose(-1, -2)], -1).to(torch.float16), E


def quantize_stage(E):
    """Scales and codes of the standalone quantize given the residual (leapquant/kernels.py:2218-2229, true divisions)."""
    V = E.shape[-2]
    sk = torch.clamp(torch.sqrt(E.abs().sum(-2) / V), min=EPS)
    sv = torch.clamp((E / sk[..., None, :]).abs().amax(-1), min=EPS)
    code = torch.clamp(torch.round(E / (sk[..., None, :] * sv[..., :, None]) * QMAX), -QMAX, QMAX).to(torch.int8)
    return sk, sv, code


def quantize(S0, Sq, Sk, Sv, UQ, Wbuf, Pbuf, hcnt, Q0, idx, iters=1):
    """fp32 slots idx of S0 [NS,HV,V,K] -> 8-bit checkpoint in the same slots, window reset (leapquant/kernels.py:2126-2242)."""
    idx = idx.to(torch.int64)
    sl = idx[idx > 0]
    if sl.numel() == 0:
        return
    NS, HV, V, K = S0.shape
    S = S0[sl].reshape(-1, V, K).clone()
    code, sk, sv, uq, _ = quantize_heads(S, Q0, iters)
    n = sl.numel()
    Sq[sl] = code.reshape(n, HV, V, K)
    Sk[sl] = sk.reshape(n, HV, K)
    Sv[sl] = sv.reshape(n, HV, V)
    UQ[sl] = uq.reshape(n, HV, -1, K + V)
    Wbuf[sl] = 0.0
    Pbuf[sl] = 1.0
    hcnt[sl] = 0


def dequant_heads(q8, Sk, Sv, uq, p, Kb, Ub, w, h):
    """fp32 state of GDN heads (leapquant/kernels.py:2105-2117):
    S = (q8/127 Sk Sv + sum_r Q_r U_r^T) p + sum_{j<h} (w_j u_j) k_j^T, factors and entries added one at a time."""
    K = q8.shape[-1]
    L = Kb.shape[-2]
    uqf = uq.to(torch.float32)
    tile = _dequant_codes(q8, Sk, Sv)
    for r in range(uqf.shape[-2]):
        tile = tile + uqf[..., r, K:, None] * uqf[..., r, None, :K]
    tile = tile * p[..., None, None]
    wl = torch.where(torch.arange(L) < h[..., None], w, torch.zeros_like(w))
    Kf, Uf = Kb.to(torch.float32), Ub.to(torch.float32)
    for j in range(L):
        tile = tile + (wl[..., j, None] * Uf[..., j, :])[..., :, None] * Kf[..., j, None, :]
    return tile


def dequantize(S0, Sq, Sk, Sv, Kbuf, Ubuf, Wbuf, Pbuf, hcnt, UQ, idx):
    """GDN: materialise the fp32 state of the slots idx in place over the packed slot and reset the window
    (leapquant/kernels.py:2041-2123, kda=False branch; the kda=True branch is dead code in the reference)."""
    idx = idx.to(torch.int64)
    sl = idx[idx > 0]
    if sl.numel() == 0:
        return
    S = dequant_heads(Sq[sl].clone(), Sk[sl].clone(), Sv[sl].clone(), UQ[sl].clone(), Pbuf[sl][..., 0], Kbuf[sl], Ubuf[sl],
                      Wbuf[sl], hcnt[sl].to(torch.int64))
    S0[sl] = S
    Wbuf[sl] = 0.0
    Pbuf[sl] = 1.0
    hcnt[sl] = 0


def lowrank_factor(x, r, iters=3, Q0=None):
    """x [..., K, V] fp32 -> U [..., K, r], Q [..., V, r]: `iters` rounds of P = x Q -> MGS, Q = x^T P -> MGS, then
    U = x Q, from Q0 = randn(V, r) seeded 0 (leapquant/kernels.py:2246-2331)."""
    *lead, K, V = x.shape
    Q0 = make_q0(V, r) if Q0 is None else Q0
    xf = x.reshape(-1, K, V).to(torch.float32)
    Q = Q0[None].expand(xf.shape[0], -1, -1).clone()
    for _ in range(iters):
        P = mgs(torch.einsum("nkv,nvr->nkr", xf, Q))
        Q = mgs(torch.einsum("nkv,nkr->nvr", xf, P))
    U = torch.einsum("nkv,nvr->nkr", xf, Q)
    return U.reshape(*lead, K, r), Q.reshape(*lead, V, r)


# --------------------------------------------------------------------------------------------------------------
# a9: KDA prefill round trip (torch code in the reference; pinned by tests/golden)
# --------------------------------------------------------------------------------------------------------------
def kda_rebuild(Sq, Sk, Sv, UQ, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, sl):
    """S = exp(P) (Q U^T + deq) + sum_j w_j u_j (x) (k_j D_j), D = flip(cumprod(flip(E))) / E with E = 1 for j >= h
    (leapquant/state.py:118-128)."""
    K = Sq.shape[-1]
    L = Kbuf.shape[2]
    uq = UQ[sl].to(torch.float32)
    S0 = (torch.einsum("nhrv,nhrc->nhvc", uq[..., K:], uq[..., :K])
          + Sq[sl].to(torch.float32) * (Sk[sl][..., None, :] / 127.0) * Sv[sl][..., :, None])
    E = Gbuf[sl].to(torch.float32)
    h = hcnt[sl]
    E = torch.where(torch.arange(L)[None, None, :, None] < h[..., None, None], E, torch.ones_like(E))
    D = torch.flip(torch.cumprod(torch.flip(E, [2]), 2), [2]) / E
    kdec = Kbuf[sl].to(torch.float32) * D
    return (torch.exp(Pbuf[sl])[..., None, :] * S0
            + torch.einsum("nhj,nhjv,nhjc->nhvc", Wbuf[sl], Ubuf[sl].to(torch.float32), kdec))


def kda_checkpoint_from_factors(S, U, Q):
    """Codes, scales and fp16 factors of the KDA checkpoint given the rank-R factors (leapquant/state.py:135-141).
    S [n,HV,V,K]; U [n,HV,K,R]; Q [n,HV,V,R]."""
    Uh, Qh = U.half(), Q.half()
    res = S - (Qh.float() @ Uh.float().transpose(-1, -2))
    sk = torch.sqrt(res.abs().mean(-2)).clamp_min(1e-12)
    sv = (res.abs() / sk[..., None, :]).amax(-1).clamp_min(1e-12)
    code = torch.clamp(torch.round(res / (sk[..., None, :] * sv[..., :, None]) * 127.0), -127, 127).to(torch.int8)
    uq = torch.cat([Uh.transpose(-1, -2), Qh.transpose(-1, -2)], -1)
    return code, sk, sv, uq


def kda_checkpoint(ssm, Sq, Sk, Sv, UQ, Wbuf, Pbuf, Gbuf, hcnt, sl, R):
    """8-bit checkpoint of the fp32 KDA states in the slots sl (leapquant/state.py:130-142)."""
    S = ssm[sl].to(torch.float32).clone()
    U, Q = lowrank_factor(S.transpose(-1, -2), R)
    code, sk, sv, uq = kda_checkpoint_from_factors(S, U, Q)
    Sq[sl] = code
    Sk[sl] = sk
    Sv[sl] = sv
    UQ[sl] = uq
    Wbuf[sl] = 0.0
    Pbuf[sl] = 0.0
    Gbuf[sl] = 1.0
    hcnt[sl] = 0


# --------------------------------------------------------------------------------------------------------------
# full dequantised state (for parity / accuracy checks) and the unquantised fp32 recurrences
# --------------------------------------------------------------------------------------------------------------
def full_state(Sq, Sk, Sv, UQ, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, sl, kda):
    """The live fp32 state [n, HV, V, K] represented by checkpoint + window, without touching anything."""
    sl = sl.to(torch.int64)
    if kda:
        return kda_rebuild(Sq, Sk, Sv, UQ, Kbuf, Ubuf, Wbuf, Pbuf, Gbuf, hcnt, sl)
    return dequant_heads(Sq[sl], Sk[sl], Sv[sl], UQ[sl], Pbuf[sl][..., 0], Kbuf[sl], Ubuf[sl], Wbuf[sl],
                         hcnt[sl].to(torch.int64))


def fp32_gdn_recurrence(S, q, k, v, alpha, beta, scale=None):
    """Unquantised gated delta rule, one token: S [.., V, K] <- alpha S + beta (v - alpha S k) k^T; o = S q.
    q, k are raw (l2-normalised here as in the kernels); returns o and updates S in place."""
    K = S.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    qn = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6) * scale
    kn = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    S.mul_(alpha[..., None, None])
    u = beta[..., None] * (v - torch.einsum("...vc,...c->...v", S, kn))
    S.add_(u[..., :, None] * kn[..., None, :])
    return torch.einsum("...vc,...c->...v", S, qn)


def fp32_kda_recurrence(S, q, k, v, alpha, beta, scale=None):
    """Unquantised KDA, one token: S <- S diag(alpha) + beta (v - S diag(alpha) k) k^T with alpha [.., K]; o = S q."""
    K = S.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    qn = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6) * scale
    kn = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    S.mul_(alpha[..., None, :])
    u = beta[..., None] * (v - torch.einsum("...vc,...c->...v", S, kn))
    S.add_(u[..., :, None] * kn[..., None, :])
    return torch.einsum("...vc,...c->...v", S, qn)


# --------------------------------------------------------------------------------------------------------------
# causal conv1d update that precedes the decode step in the serving engine (not part of the reference package: the plugin
# calls vLLM's Triton kernel, call sites leapquant/vllm/gdn.py:32 and leapquant/vllm/glm.py:72; vllm==0.30.0 is not vendored)
# --------------------------------------------------------------------------------------------------------------
def causal_conv1d_update(x, conv_state, weight, bias, idx):
    """Single-token causal conv1d update with SiLU, restating the published algorithm of vLLM's
    `causal_conv1d_update` (vllm/model_executor/layers/mamba/ops/causal_conv1d.py, `_causal_conv1d_update_kernel`):
    per row n with slot = idx[n] > 0 and channel c: window = (state[slot, c, 0 .. W-2], x[n, c]); every product
    weight[c, t] * window[t] is a bf16 x bf16 product rounded to bf16; they are added to the bias in fp32, taps in order;
    out = acc / (1 + exp(-acc)) rounded to bf16; state[slot, c] <- window[1:].  x bf16 [N, C], conv_state bf16 (slot, channel,
    W - 1) (any strides; updated in place), weight bf16 [C, W], bias bf16 [C] or None.  Rows with idx <= 0 are skipped and their
    output rows are left as they are (zeros here).  Parity at this boundary is unpinned by the reference: its repository holds
    no test or vector for it."""
    N, C = x.shape[0], weight.shape[0]
    W = weight.shape[1]
    out = torch.zeros(N, C, dtype=torch.bfloat16)
    idx = idx.to(torch.int64)
    rows = torch.nonzero(idx > 0).flatten()
    if rows.numel() == 0:
        return out
    sl = idx[rows]
    win = torch.cat([conv_state[sl].to(torch.float32), x[rows, :C].to(torch.float32)[..., None]], -1)      # [n, C, W]
    acc = (bias.to(torch.float32) if bias is not None else torch.zeros(C))[None].expand(rows.numel(), C).clone()
    wf = weight.to(torch.float32)
    for t in range(W):
        acc = acc + _bf16(win[..., t] * wf[None, :, t])
    out[rows] = (acc / (1.0 + torch.exp(-acc))).to(torch.bfloat16)
    conv_state[sl] = win[..., 1:].to(torch.bfloat16)
    return out


# --------------------------------------------------------------------------------------------------------------
# synthetic workloads (the seeded distributions of the benchmark configurations)
# --------------------------------------------------------------------------------------------------------------
def synth_inputs(N, H, HV, K, V, steps, seed, kda=False, dtype=torch.bfloat16):
    """q, k ~ N(0,1) l2-normalised per head, v ~ N(0,1), b ~ N(0,1) (beta = sigmoid b), a ~ N(0,1) with A_log = 0 and
    dt_bias = 0 so that alpha = exp(-softplus a).  Returns per-step tensors stacked on dim 0."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(steps, N, H, K, generator=g)
    k = torch.randn(steps, N, H, K, generator=g)
    q = q / q.norm(dim=-1, keepdim=True)
    k = k / k.norm(dim=-1, keepdim=True)
    v = torch.randn(steps, N, HV, V, generator=g)
    mixed = torch.cat([q.reshape(steps, N, -1), k.reshape(steps, N, -1), v.reshape(steps, N, -1)], -1).to(dtype)
    a = torch.randn(steps, N, HV, K if kda else 1, generator=g).to(dtype)
    if not kda:
        a = a[..., 0]
    b = torch.randn(steps, N, HV, generator=g).to(dtype)
    A_log = torch.zeros(HV)
    dt_bias = torch.zeros(HV, K) if kda else torch.zeros(HV)
    return mixed, a, b, A_log, dt_bias


def outlier_states(n, HV, V, K, seed, frac=0.01, gain=50.0):
    """fp32 states ~ N(0,1) with `frac` of the rows and of the columns scaled by `gain` (seeded choice)."""
    g = torch.Generator().manual_seed(seed)
    S = torch.randn(n, HV, V, K, generator=g)
    nr, nc = max(1, int(round(frac * V))), max(1, int(round(frac * K)))
    for i in range(n):
        for hh in range(HV):
            S[i, hh, torch.randperm(V, generator=g)[:nr], :] *= gain
            S[i, hh, :, torch.randperm(K, generator=g)[:nc]] *= gain
    return S
