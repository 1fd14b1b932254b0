"""End-to-end tensor-parallel decode harness: a random-init hybrid model of the shape of the benchmark's last configuration
-- hidden 4096, 32 layers in a 3:1 interleave of Gated DeltaNet layers (16 key / 32 value heads of 128) and gated
full-attention layers (32 query / 8 KV heads of 128), SwiGLU MLP 12288, vocabulary 151 936 -- sharded over the GPUs of one
box, one process per GPU, with an NCCL all-reduce after every out-projection and MLP.

It exists to compare, end to end and on identical weights and prompts, the 8-bit recurrent state of this package
(`state="int8"`: conv1d update + decode step + flush as ONE launch per layer and step) with the engine's fp32 state
(`state="fp32"`: vLLM's own conv1d-update and packed-decode kernels on an fp32 state, where that vLLM is importable; else
flash-linear-attention's recurrent kernel).  Everything that is not the recurrent state path -- projections, attention
over a KV cache, MLP, norms, sampling, the chunked prefill of the delta rule -- is plain PyTorch or library code: it is the
same in both arms and is not what this package accelerates.  The reference plugs into vLLM for this (leapquant/vllm/gdn.py);
the vLLM it pins is not the one of this image, so the model loop is written out here.

The only communication is the tensor-parallel all-reduce (and the arg-max exchange of the sharded LM head); the recurrent
state of a layer lives on the rank that owns its heads and never crosses a link.
"""
import math
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F


class HybridConfig:
    hidden = 4096
    layers = 32
    full_attention_every = 4          # layers 3, 7, 11, ... are full attention, the others Gated DeltaNet
    gdn_key_heads, gdn_value_heads, gdn_dim = 16, 32, 128
    attn_q_heads, attn_kv_heads, attn_dim = 32, 8, 128
    mlp = 12288
    vocab = 151936
    conv_width = 4
    window, rank = 64, 4              # LeapQuant: window length, Compensator Tokens
    rope_base = 10000.0

    def __init__(self, **kw):
        for k, v in kw.items():
            if not hasattr(self, k):
                raise AttributeError(k)
            setattr(self, k, v)


def _w(shape, seed, device, std=0.02):
    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * std).to(torch.bfloat16)


def rms_norm(x, weight, eps=1e-6):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * weight


class HybridTP:
    """One rank's shard of the model, its KV cache, its recurrent states and its prefill / decode loops."""

    def __init__(self, cfg, rank, world, device, state, batch, max_len):
        assert state in ("int8", "fp32")
        self.cfg, self.rank, self.world, self.dev, self.state_mode = cfg, rank, world, device, state
        self.B, self.max_len = batch, max_len
        c = cfg
        assert c.gdn_key_heads % world == 0 and c.attn_kv_heads % world == 0 and c.mlp % world == 0 and c.vocab % world == 0
        self.H, self.HV, self.D = c.gdn_key_heads // world, c.gdn_value_heads // world, c.gdn_dim
        self.QH, self.KVH, self.AD = c.attn_q_heads // world, c.attn_kv_heads // world, c.attn_dim
        self.C = 2 * self.H * self.D + self.HV * self.D          # local q | k | v channels of a GDN layer
        self.mlp_l, self.vocab_l = c.mlp // world, c.vocab // world
        hid = c.hidden
        s = lambda l, k: 1000 * l + 10 * k + 100000 * rank       # weight seeds: identical in both arms, distinct per shard
        self.embed = _w((c.vocab, hid), 7, device)               # replicated (same seed on every rank)
        self.lm_head = _w((self.vocab_l, hid), 8 + 100000 * rank, device)
        self.final_norm = torch.ones(hid, dtype=torch.bfloat16, device=device)
        self.layers = []
        for l in range(c.layers):
            p = {"kind": "attn" if (l + 1) % c.full_attention_every == 0 else "gdn",
                 "norm1": torch.ones(hid, dtype=torch.bfloat16, device=device),
                 "norm2": torch.ones(hid, dtype=torch.bfloat16, device=device),
                 "gate_up": _w((2 * self.mlp_l, hid), s(l, 5), device), "down": _w((hid, self.mlp_l), s(l, 6), device)}
            if p["kind"] == "gdn":
                p["in_qkvz"] = _w((self.C + self.HV * self.D, hid), s(l, 1), device)      # q | k | v | z
                p["in_ba"] = _w((2 * self.HV, hid), s(l, 2), device, std=0.2)
                p["conv_w"] = _w((self.C, c.conv_width), s(l, 3), device, std=0.3)
                p["conv_b"] = torch.zeros(self.C, dtype=torch.bfloat16, device=device)
                p["A_log"] = torch.zeros(self.HV, device=device)
                p["dt_bias"] = torch.zeros(self.HV, device=device)
                p["gnorm"] = torch.ones(self.D, dtype=torch.bfloat16, device=device)
                p["out"] = _w((hid, self.HV * self.D), s(l, 4), device)
                # recurrent state [slots, HV, V, K] fp32 (slot 0 is the null slot) and conv state [slots, width - 1, C]
                p["ssm"] = torch.zeros(batch + 1, self.HV, self.D, self.D, device=device)
                p["conv"] = torch.zeros(batch + 1, c.conv_width - 1, self.C, dtype=torch.bfloat16, device=device)
            else:
                p["q"] = _w((2 * self.QH * self.AD, hid), s(l, 1), device)                # q | gate
                p["kv"] = _w((2 * self.KVH * self.AD, hid), s(l, 2), device)
                p["out"] = _w((hid, self.QH * self.AD), s(l, 4), device)
                p["kc"] = torch.zeros(batch, self.KVH, max_len, self.AD, dtype=torch.bfloat16, device=device)
                p["vc"] = torch.zeros_like(p["kc"])
            self.layers.append(p)
        half = self.AD // 2
        inv = 1.0 / (c.rope_base ** (torch.arange(half, device=device).float() / half))
        ang = torch.arange(max_len, device=device).float()[:, None] * inv[None]
        self.cos, self.sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
        self.slots = torch.arange(1, batch + 1, dtype=torch.int32, device=device)
        self.fp32_kernels = None
        if state == "fp32":
            self.fp32_kernels = self._find_fp32_kernels()
        self.lq = {}
        self.kv_attention = self._find_kv_attention()

    def _find_kv_attention(self):
        """Decode attention over the KV cache from a library when one runs on this device (flash_attn's kv-cache kernel:
        appends the new key / value and attends in one call); None = torch's scaled_dot_product_attention with a mask.
        Attention is not part of the path this package accelerates: both arms of the comparison use the same one."""
        try:
            from flash_attn import flash_attn_with_kvcache
            kc = torch.zeros(1, 16, self.KVH, self.AD, dtype=torch.bfloat16, device=self.dev)
            q = torch.zeros(1, 1, self.QH, self.AD, dtype=torch.bfloat16, device=self.dev)
            kn = torch.zeros(1, 1, self.KVH, self.AD, dtype=torch.bfloat16, device=self.dev)
            flash_attn_with_kvcache(q, kc, kc.clone(), k=kn, v=kn, cache_seqlens=torch.zeros(1, dtype=torch.int32, device=self.dev),
                                    causal=True)
            torch.cuda.synchronize()
            return flash_attn_with_kvcache
        except Exception:
            return None

    # ---- pieces ----
    def all_reduce(self, x):
        if self.world > 1:
            dist.all_reduce(x)
        return x

    def rope(self, x, pos):
        """x [..., T, AD] with positions pos [T] (or [B, 1] for decode)."""
        cos, sin = self.cos[pos], self.sin[pos]
        x1, x2 = x[..., : self.AD // 2], x[..., self.AD // 2:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)

    def mlp(self, p, x):
        gu = F.linear(x, p["gate_up"])
        g, u = gu.split(self.mlp_l, -1)
        return self.all_reduce(F.linear(F.silu(g) * u, p["down"]))

    @staticmethod
    def _find_fp32_kernels():
        try:
            from vllm.model_executor.layers.fla.ops.fused_recurrent import fused_recurrent_gated_delta_rule_packed_decode as dec
            from vllm.model_executor.layers.mamba.ops.causal_conv1d import causal_conv1d_update as conv
            return ("vllm", conv, dec)
        except Exception:
            from fla.ops.gated_delta_rule import fused_recurrent_gated_delta_rule as dec
            return ("fla", None, dec)

    def lq_state(self, l):
        if l not in self.lq:
            from .state import LeapQuantState
            self.lq[l] = LeapQuantState(self.layers[l]["ssm"], self.H, L=self.cfg.window, R=self.cfg.rank, nmax=self.B)
        return self.lq[l]

    # ---- prefill: whole prompts, a few sequences at a time ----
    @torch.no_grad()
    def prefill(self, tokens, seqs_per_pass=8):
        """tokens [B, T] -> next token ids [B] (greedy).  Fills the KV caches, the conv states and the recurrent states."""
        from fla.ops.gated_delta_rule import chunk_gated_delta_rule
        B, T = tokens.shape
        last = torch.empty(B, self.cfg.hidden, dtype=torch.bfloat16, device=self.dev)
        pos = torch.arange(T, device=self.dev)
        for b0 in range(0, B, seqs_per_pass):
            b1 = min(B, b0 + seqs_per_pass)
            n = b1 - b0
            x = self.embed[tokens[b0:b1]]                                            # [n, T, hid]
            for l, p in enumerate(self.layers):
                h = rms_norm(x, p["norm1"])
                if p["kind"] == "gdn":
                    qkvz = F.linear(h, p["in_qkvz"])
                    raw, z = qkvz[..., : self.C], qkvz[..., self.C:]
                    ba = F.linear(h, p["in_ba"])
                    b_, a_ = ba[..., : self.HV], ba[..., self.HV:]
                    p["conv"][b0 + 1:b1 + 1] = raw[:, T - (self.cfg.conv_width - 1):, :]                  # last inputs, (slot, tap, channel)
                    xc = F.conv1d(F.pad(raw.transpose(1, 2), (self.cfg.conv_width - 1, 0)), p["conv_w"][:, None, :], p["conv_b"],
                                  groups=self.C)
                    mixed = F.silu(xc).transpose(1, 2)
                    q, k, v = mixed.split([self.H * self.D, self.H * self.D, self.HV * self.D], -1)
                    rep = self.HV // self.H
                    q = q.reshape(n, T, self.H, self.D).repeat_interleave(rep, 2)
                    k = k.reshape(n, T, self.H, self.D).repeat_interleave(rep, 2)
                    v = v.reshape(n, T, self.HV, self.D)
                    g = -torch.exp(p["A_log"]) * F.softplus(a_.float() + p["dt_bias"])
                    beta = torch.sigmoid(b_.float()).to(torch.bfloat16)
                    o, S = chunk_gated_delta_rule(q, k, v, g, beta, scale=self.D ** -0.5, output_final_state=True,
                                                  use_qk_l2norm_in_kernel=True)
                    p["ssm"][b0 + 1:b1 + 1] = S.transpose(-1, -2).float()            # fla keeps [.., K, V]; the engine's slot is [V, K]
                    o = rms_norm(o, p["gnorm"]) * F.silu(z.reshape(n, T, self.HV, self.D))
                    y = F.linear(o.reshape(n, T, -1), p["out"])
                else:
                    qg = F.linear(h, p["q"]).reshape(n, T, 2, self.QH, self.AD)
                    kv = F.linear(h, p["kv"]).reshape(n, T, 2, self.KVH, self.AD)
                    q = self.rope(qg[:, :, 0].transpose(1, 2), pos)
                    k = self.rope(kv[:, :, 0].transpose(1, 2), pos)
                    v = kv[:, :, 1].transpose(1, 2)
                    p["kc"][b0:b1, :, :T] = k
                    p["vc"][b0:b1, :, :T] = v
                    o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
                    o = o.transpose(1, 2) * torch.sigmoid(qg[:, :, 1].float()).to(o.dtype)
                    y = F.linear(o.reshape(n, T, -1), p["out"])
                x = x + self.all_reduce(y)
                x = x + self.mlp(p, rms_norm(x, p["norm2"]))
            last[b0:b1] = x[:, -1]
        if self.state_mode == "int8":
            for l, p in enumerate(self.layers):
                if p["kind"] == "gdn":
                    self.lq_state(l).quantize(p["ssm"], self.slots)
        return self.sample(last)

    def sample(self, x):
        """Greedy token of the sharded LM head: local arg-max, then the best of all ranks."""
        logits = F.linear(rms_norm(x, self.final_norm), self.lm_head).float()
        val, idx = logits.max(-1)
        idx = idx + self.rank * self.vocab_l
        if self.world > 1:
            vals = [torch.empty_like(val) for _ in range(self.world)]
            idxs = [torch.empty_like(idx) for _ in range(self.world)]
            dist.all_gather(vals, val)
            dist.all_gather(idxs, idx)
            best = torch.stack(vals).argmax(0)
            idx = torch.stack(idxs).gather(0, best[None])[0]
        return idx

    # ---- one decode step of the whole batch ----
    @torch.no_grad()
    def decode_step(self, tokens, pos):
        """tokens [B] int64, pos [B] int64 (their positions) -> next tokens [B].  No host synchronisation: capturable."""
        B = self.B
        x = self.embed[tokens]
        for l, p in enumerate(self.layers):
            h = rms_norm(x, p["norm1"])
            if p["kind"] == "gdn":
                qkvz = F.linear(h, p["in_qkvz"])
                raw, z = qkvz[:, : self.C], qkvz[:, self.C:]
                ba = F.linear(h, p["in_ba"])
                b_, a_ = ba[:, : self.HV].contiguous(), ba[:, self.HV:].contiguous()
                o = torch.empty(B, self.HV, self.D, dtype=torch.bfloat16, device=self.dev)
                conv_view = p["conv"].transpose(-1, -2)                                   # (slot, channel, tap)
                if self.state_mode == "int8":
                    self.lq_state(l).decode_conv(p["ssm"], raw, conv_view, p["conv_w"], p["conv_b"], a_, b_, p["A_log"], p["dt_bias"],
                                                 self.slots, o)
                else:
                    kind, conv, dec = self.fp32_kernels
                    if kind == "vllm":
                        mixed = conv(raw.contiguous(), conv_view, p["conv_w"], p["conv_b"], "silu", conv_state_indices=self.slots)
                        dec(mixed_qkv=mixed, a=a_, b=b_, A_log=p["A_log"], dt_bias=p["dt_bias"], scale=self.D ** -0.5,
                            initial_state=p["ssm"], out=o.unsqueeze(1), ssm_state_indices=self.slots, use_qk_l2norm_in_kernel=True)
                    else:
                        win = torch.cat([p["conv"][1:], raw[:, None, :]], 1)              # [B, width, C]
                        p["conv"][1:] = win[:, 1:]
                        mixed = F.silu((win.float() * p["conv_w"].t().float()[None]).sum(1) + p["conv_b"].float()).to(torch.bfloat16)
                        q, k, v = mixed.split([self.H * self.D, self.H * self.D, self.HV * self.D], -1)
                        rep = self.HV // self.H
                        q = q.reshape(B, 1, self.H, self.D).repeat_interleave(rep, 2)
                        k = k.reshape(B, 1, self.H, self.D).repeat_interleave(rep, 2)
                        g = (-torch.exp(p["A_log"]) * F.softplus(a_.float() + p["dt_bias"]))[:, None]
                        oo, S = dec(q, k, v.reshape(B, 1, self.HV, self.D), g=g, beta=torch.sigmoid(b_.float()).to(torch.bfloat16)[:, None],
                                    scale=self.D ** -0.5, initial_state=p["ssm"][1:].transpose(-1, -2).contiguous(),
                                    output_final_state=True, use_qk_l2norm_in_kernel=True)
                        p["ssm"][1:] = S.transpose(-1, -2)
                        o = oo[:, 0]
                o = rms_norm(o, p["gnorm"]) * F.silu(z.reshape(B, self.HV, self.D))
                y = F.linear(o.reshape(B, -1), p["out"])
            else:
                qg = F.linear(h, p["q"]).reshape(B, 2, self.QH, self.AD)
                kv = F.linear(h, p["kv"]).reshape(B, 2, self.KVH, self.AD)
                q = self.rope(qg[:, 0], pos[:, None])                                     # [B, QH, AD]
                k = self.rope(kv[:, 0], pos[:, None])
                if self.kv_attention is not None:
                    o = self.kv_attention(q[:, None], p["kc"].transpose(1, 2), p["vc"].transpose(1, 2), k=k[:, None], v=kv[:, 1][:, None],
                                          cache_seqlens=pos.to(torch.int32), causal=True)[:, 0]
                else:
                    ar = torch.arange(B, device=self.dev)
                    p["kc"][ar, :, pos] = k
                    p["vc"][ar, :, pos] = kv[:, 1]
                    mask = (torch.arange(self.max_len, device=self.dev)[None] <= pos[:, None])[:, None, None, :]
                    o = F.scaled_dot_product_attention(q[:, :, None], p["kc"], p["vc"], attn_mask=mask, enable_gqa=True)[:, :, 0]
                o = o * torch.sigmoid(qg[:, 1].float()).to(o.dtype)
                y = F.linear(o.reshape(B, -1), p["out"])
            x = x + self.all_reduce(y)
            x = x + self.mlp(p, rms_norm(x, p["norm2"]))
        return self.sample(x)


def run_generation(cfg, state, batch, prompt_len, new_tokens, seed=0, use_graph=True):
    """Greedy generation on random prompts; returns a dict with times (device-timed, max over ranks) and throughput."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    dev = torch.device("cuda", torch.cuda.current_device())
    model = HybridTP(cfg, rank, world, dev, state, batch, prompt_len + new_tokens + 1)
    g = torch.Generator(device="cpu").manual_seed(seed)
    prompts = torch.randint(0, cfg.vocab, (batch, prompt_len), generator=g).to(dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)
    e0, e1, e2 = ev(), ev(), ev()
    model.prefill(prompts[:1, :min(prompt_len, 128)])          # warm-up: compiles the library kernels of the prefill (slot 1 is rewritten below)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0.record()
    tok = model.prefill(prompts)
    e1.record()
    pos = torch.full((batch,), prompt_len, dtype=torch.int64, device=dev)
    first = tok.clone()
    graph, mode = None, "eager"
    s_tok, s_pos = tok.clone(), pos.clone()
    if use_graph:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):                                                   # warm-up outside the capture (Triton compiles, NCCL)
                    s_next = model.decode_step(s_tok, s_pos)
                    s_tok.copy_(s_next)
                    s_pos.add_(1)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                s_next = model.decode_step(s_tok, s_pos)
                s_tok.copy_(s_next)
                s_pos.add_(1)
            mode = "cuda_graph"
            done = 2
        except Exception as e:                                                       # keep going without the graph
            graph, mode, done = None, "eager (capture failed: %s)" % str(e).splitlines()[0][:120], 0
            s_tok, s_pos = tok.clone(), pos.clone()
    else:
        done = 0
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e1b = ev()
    e1b.record()
    steps = new_tokens - done - (1 if graph is not None else 0)
    for _ in range(steps):
        if graph is not None:
            graph.replay()
        else:
            s_next = model.decode_step(s_tok, s_pos)
            s_tok.copy_(s_next)
            s_pos.add_(1)
    e2.record()
    torch.cuda.synchronize()
    t_prefill, t_decode = e0.elapsed_time(e1) * 1e-3, e1b.elapsed_time(e2) * 1e-3
    t = torch.tensor([t_prefill, t_decode], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    t_prefill, t_decode = float(t[0]), float(t[1])
    return {"state": state, "fp32_kernels": model.fp32_kernels[0] if model.fp32_kernels else None, "decode_mode": mode,
            "attention": "flash_attn_with_kvcache" if model.kv_attention is not None else "torch sdpa, masked",
            "prefill_s": t_prefill, "decode_s": t_decode, "decode_steps_timed": steps, "ms_per_decode_step": 1e3 * t_decode / max(steps, 1),
            "decode_tokens_per_s": batch * steps / t_decode if steps else None, "first_tokens": first[:8].tolist(),
            "last_tokens": s_tok[:8].tolist(),
            "state_bytes_per_gpu": sum(p["ssm"].numel() * 4 for p in model.layers if p["kind"] == "gdn")}
