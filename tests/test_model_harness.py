"""The prefill harness around the LUCID solve (bench_lucid_model.py): sliding-window helper against a dense
mask on the CPU, and a reduced-size model on the GPU (both variants finite, LUCID layers change the result,
the solve inside the model equals the oracle on the same K/V)."""
import importlib

import pytest
import torch


def test_sliding_window_matches_dense_mask_cpu():
    m = importlib.import_module("bench_lucid_model")
    torch.manual_seed(0)
    B, Hq, Hkv, N, D, W = 1, 4, 2, 512, 16, 128
    q, k, v = torch.randn(B, Hq, N, D), torch.randn(B, Hkv, N, D), torch.randn(B, Hkv, N, D)
    out = m.sliding_window_attention(q, k, v, W)
    i, j = torch.arange(N)[:, None], torch.arange(N)[None, :]
    ref = torch.nn.functional.scaled_dot_product_attention(
        q, k.repeat_interleave(2, 1), v.repeat_interleave(2, 1), attn_mask=(j <= i) & (j > i - W))
    assert float((out - ref).abs().max()) < 1e-5


@pytest.mark.gpu
def test_reduced_model_runs_both_variants(monkeypatch):
    m = importlib.import_module("bench_lucid_model")
    monkeypatch.setitem(m.CFG, "layers", 6)
    monkeypatch.setitem(m.CFG, "hidden", 512)
    monkeypatch.setitem(m.CFG, "mlp", 1024)
    monkeypatch.setitem(m.CFG, "vocab", 4096)
    monkeypatch.setitem(m.CFG, "window", 256)
    dev = torch.device("cuda", 0)
    model = m.Model(dev)
    ids = torch.randint(0, 4096, (1, 1024), device=dev)
    a = model.prefill(ids, lucid=False)
    tap = []
    b = model.prefill(ids, lucid=True, tap=tap)
    assert torch.isfinite(a.float()).all() and torch.isfinite(b.float()).all()
    assert not torch.equal(a, b)          # the one global layer (the 6th) went through the solve
    # the solve inside the model against the oracle on the very K/V it was handed (strided BSHD views of the
    # model's BHSD tensors, key scale folded into the kernels)
    from oracle import lucid_oracle as orc

    assert [t[0] for t in tap] == [5]
    _, k, v, v_prime, ks = tap[0]
    assert not k.is_contiguous() and k.shape == (1, 1024, 4, 128)
    ref = orc.forward_sub_blockwise(k.double() * ks, v.double())
    assert orc.rel_err(v_prime, ref) < 0.01
