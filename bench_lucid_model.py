#!/usr/bin/env python
"""Prefill throughput of a Gemma-3-4B-style decoder with LUCID applied to the K/V of its global layers,
against the same model with plain softmax attention everywhere.

Counterpart of the reference's bench_lucid_model.py (its model: :139-256, layer pattern :276-297, LUCID
call site `_lucid_solve` :164-170,189-193), built to the configuration the benchmark names rather than to
the reference's smaller one: 34 layers, every 6th one global (5 global layers with LUCID on K/V, 29
sliding-window softmax layers, window 1024), hidden 2560, 8 query heads / 4 KV heads (GQA 2:1),
head_dim 128, GeGLU MLP 10240, vocabulary 262144, RMSNorm, RoPE; batch 1, random-init bf16 weights,
uniform-random token ids (synthetic: no dataset or checkpoint is involved).

Everything around the LUCID solve is plain PyTorch (cuBLAS GEMMs, torch SDPA): plumbing that is identical
in both variants, so that the difference between the two is the cost of the solve and its call-site glue.

    python bench_lucid_model.py [--seqlens 2048 8192 32768 65536] [--iters 5] [--vprime-residency]

Prints one JSON line per sequence length: tokens/s of both variants and the LUCID overhead.  With
--vprime-residency it also times, per sequence length, a global layer's attention call straight after the
solve that produced V' (V' as warm in the L2 cache as the solve leaves it) and after the L2 has been
overwritten (V' read back from HBM): the difference is what keeping V' resident for, or fusing its
production with, the attention of the same layer (the step after the solve at the reference's call site,
bench_lucid_model.py:189-193) could save at most.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CFG = dict(layers=34, global_every=6, hidden=2560, q_heads=8, kv_heads=4, head_dim=128, mlp=10240,
           vocab=262144, window=1024, rope_base=10000.0)


def rms_norm(x, w, eps=1e-6):
    return F.rms_norm(x, (x.shape[-1],), w, eps)


def rope(x, cos, sin):
    # x: (B, H, N, D); rotate half
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1)


def sliding_window_attention(q, k, v, window):
    """Causal attention restricted to the last `window` keys, as block-local attention: queries of chunk c
    see chunk c-1 and chunk c through one shared (window x 2*window) band mask.  q: (B, Hq, N, D),
    k, v: (B, Hkv, N, D)."""
    B, Hq, N, D = q.shape
    if N <= window:
        return F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
    assert N % window == 0
    C = N // window
    Hkv = k.shape[1]
    # the first chunk has no predecessor: plain causal attention
    first = F.scaled_dot_product_attention(q[:, :, :window], k[:, :, :window], v[:, :, :window], is_causal=True,
                                           enable_gqa=True)
    qc = q[:, :, window:].reshape(B, Hq, C - 1, window, D).permute(0, 2, 1, 3, 4).reshape(B * (C - 1), Hq, window, D)

    def prev_and_cur(t):
        tc = t.reshape(B, Hkv, C, window, D)
        both = torch.cat((tc[:, :, :-1], tc[:, :, 1:]), dim=3)     # (B, Hkv, C-1, 2*window, D)
        return both.permute(0, 2, 1, 3, 4).reshape(B * (C - 1), Hkv, 2 * window, D)

    kc, vc = prev_and_cur(k), prev_and_cur(v)
    qi = torch.arange(window, device=q.device)[:, None] + window
    kj = torch.arange(2 * window, device=q.device)[None, :]
    band = ((kj <= qi) & (kj > qi - window))[None, None]          # (1, 1, window, 2*window), shared by all chunks
    rest = F.scaled_dot_product_attention(qc, kc, vc, attn_mask=band, enable_gqa=True)
    rest = rest.reshape(B, C - 1, Hq, window, D).permute(0, 2, 1, 3, 4).reshape(B, Hq, N - window, D)
    return torch.cat((first, rest), dim=2)


class Model:
    def __init__(self, device, dtype=torch.bfloat16, seed=0):
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        c = CFG
        def w(*shape, scale=None):
            scale = scale if scale is not None else 1.0 / math.sqrt(shape[-1])
            return (torch.randn(*shape, device=device, dtype=torch.float32, generator=g) * scale).to(dtype)
        self.embed = w(c["vocab"], c["hidden"], scale=1.0)
        self.layers = []
        qd, kvd = c["q_heads"] * c["head_dim"], c["kv_heads"] * c["head_dim"]
        for _ in range(c["layers"]):
            self.layers.append(dict(
                n1=torch.ones(c["hidden"], device=device, dtype=dtype),
                n2=torch.ones(c["hidden"], device=device, dtype=dtype),
                wqkv=w(qd + 2 * kvd, c["hidden"]), wo=w(c["hidden"], qd),
                wgu=w(2 * c["mlp"], c["hidden"]), wd=w(c["hidden"], c["mlp"])))
        self.norm = torch.ones(c["hidden"], device=device, dtype=dtype)

    @torch.no_grad()
    def prefill(self, ids, lucid: bool, tap=None):
        """Returns the last position's logits.  `lucid`: apply the LUCID solve to K/V of the global layers.
        `tap`: a list that receives (layer index, k, v, v_prime, k_scale) of every solve, k and v being the
        BSHD views handed to it."""
        from lucid_kernels_b200.cute import _forward_sub_fwd

        c = CFG
        B, N = ids.shape
        D, Hq, Hkv = c["head_dim"], c["q_heads"], c["kv_heads"]
        x = self.embed[ids] * math.sqrt(c["hidden"])
        pos = torch.arange(N, device=ids.device, dtype=torch.float32)
        inv = c["rope_base"] ** (-torch.arange(0, D // 2, device=ids.device, dtype=torch.float32) / (D // 2))
        ang = pos[:, None] * inv[None, :]
        cos, sin = ang.cos().to(x.dtype)[None, None], ang.sin().to(x.dtype)[None, None]
        for li, L in enumerate(self.layers):
            is_global = (li + 1) % c["global_every"] == 0
            h = rms_norm(x, L["n1"])
            qkv = h @ L["wqkv"].T
            q, k, v = qkv.split((Hq * D, Hkv * D, Hkv * D), dim=-1)
            q = rope(q.reshape(B, N, Hq, D).transpose(1, 2), cos, sin)
            k = rope(k.reshape(B, N, Hkv, D).transpose(1, 2), cos, sin)
            v = v.reshape(B, N, Hkv, D).transpose(1, 2)
            if is_global:
                scale = None
                if lucid:
                    # call site of the reference (keys scaled by d^-1/4, V' = solve(k, v), attention on the
                    # scaled keys) without its glue: the BHSD-backed tensors go in as strided BSHD views, the
                    # key scale is folded into the solve and into the attention scale instead of being applied
                    # to k in a pass of its own
                    ks = D ** -0.25
                    v_prime = _forward_sub_fwd(k.transpose(1, 2), v.transpose(1, 2), k_scale=ks)
                    if tap is not None:
                        tap.append((li, k.transpose(1, 2), v.transpose(1, 2), v_prime, ks))
                    v = v_prime.transpose(1, 2)
                    scale = ks / math.sqrt(D)                          # q . (ks k) / sqrt(d)
                a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True, scale=scale)
            else:
                a = sliding_window_attention(q, k, v, c["window"])
            x = x + a.transpose(1, 2).reshape(B, N, Hq * D) @ L["wo"].T
            h = rms_norm(x, L["n2"])
            gu = h @ L["wgu"].T
            gate, up = gu.split(c["mlp"], dim=-1)
            x = x + (F.gelu(gate, approximate="tanh") * up) @ L["wd"].T
        last = rms_norm(x[:, -1], self.norm)
        return last @ self.embed.T


@torch.no_grad()
def vprime_residency_probe(N, dev, iters=10):
    """One global layer's solve followed by its attention call, at the model's head counts: attention timed
    with V' as the solve left it (warm) and after 256 MiB of other writes went through the L2 (cold)."""
    from lucid_kernels_b200.cute import _forward_sub_fwd

    c = CFG
    D, Hq, Hkv = c["head_dim"], c["q_heads"], c["kv_heads"]
    g = torch.Generator(device=dev)
    g.manual_seed(7)
    q = torch.randn(1, Hq, N, D, device=dev, dtype=torch.bfloat16, generator=g)
    k = torch.randn(1, Hkv, N, D, device=dev, dtype=torch.bfloat16, generator=g)
    v = torch.randn(1, Hkv, N, D, device=dev, dtype=torch.bfloat16, generator=g)
    ks = D ** -0.25
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    res = {}
    for name, evict in (("warm", False), ("cold", True)):
        tot = 0.0
        for it in range(iters + 2):
            vp = _forward_sub_fwd(k.transpose(1, 2), v.transpose(1, 2), k_scale=ks).transpose(1, 2)
            if evict:
                flush.fill_(it & 255)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            F.scaled_dot_product_attention(q, k, vp, is_causal=True, enable_gqa=True, scale=ks / math.sqrt(D))
            b.record()
            torch.cuda.synchronize()
            if it >= 2:
                tot += a.elapsed_time(b)
        res[name] = tot / iters
    vp_bytes = N * Hkv * D * 2
    return dict(seqlen=N, attention_ms_vprime_warm=res["warm"], attention_ms_vprime_cold=res["cold"],
                saving_ms=res["cold"] - res["warm"], vprime_bytes=vp_bytes,
                hbm_round_trip_ms_at_6_5_TBps=2 * vp_bytes / 6.5e12 * 1e3)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seqlens", type=int, nargs="+", default=[2048, 8192, 32768, 65536])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--vprime-residency", action="store_true")
    args = ap.parse_args()
    assert torch.cuda.is_available(), "needs a CUDA device"
    dev = torch.device("cuda", 0)
    model = Model(dev)
    for N in args.seqlens:
        g = torch.Generator(device=dev)
        g.manual_seed(N)
        ids = torch.randint(0, CFG["vocab"], (1, N), device=dev, generator=g)
        res = {}
        for lucid in (False, True, False, True):      # warm both variants before either is timed
            model.prefill(ids, lucid)
        for name, lucid in (("softmax", False), ("lucid", True)):
            model.prefill(ids, lucid)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(args.iters):
                out = model.prefill(ids, lucid)
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / args.iters
            res[name] = dict(ms=ms, tok_s=N / ms * 1e3, finite=bool(torch.isfinite(out.float()).all()))
        over = res["lucid"]["ms"] / res["softmax"]["ms"] - 1.0
        print(json.dumps(dict(metric="prefill_tok_s", seqlen=N, batch=1, dtype="bf16", data="synthetic",
                              config="Gemma-3-4B-style: 34 layers (5 global + LUCID, 29 sliding window 1024), "
                                     "hidden 2560, 8q/4kv heads, d 128, GeGLU 10240, vocab 262144",
                              softmax=res["softmax"], lucid=res["lucid"], lucid_overhead=over)), flush=True)
        if args.vprime_residency:
            print(json.dumps(dict(metric="vprime_residency", **vprime_residency_probe(N, dev))), flush=True)


if __name__ == "__main__":
    main()
