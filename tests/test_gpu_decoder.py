"""The decoder harness on a GPU: paged-KV row addressing and the prefill / decode paths agree.

Small layer counts of the two configured architectures.  (1) Decoding token S after a prefill of S
tokens gives the logits a prefill of S+1 tokens gives at its last position: the W8A8 linears are
row-independent and bit-exact between the GEMM and the decode kernels, so the only differences come
from PyTorch's attention kernels (tolerance written below).  (2) A scattered block table and the
identity block table give identical logits: cache rows are addressed as
block_table[pos // 16] * 16 + pos % 16 (native/src/runtime/paged_kv.h).  (3) The decode step can be
captured in a CUDA graph and replayed with updated token / position tensors."""
import numpy as np
import pytest

from tests import decoder_harness as dh

pytestmark = pytest.mark.gpu
LOGIT_TOL = 2e-3   # max |delta| / rms(logits): attention runs through different PyTorch kernels in the two paths


@pytest.fixture(scope="module")
def torch():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch


def rel(a, b):
    return float((a - b).abs().max() / b.pow(2).mean().sqrt())


@pytest.mark.parametrize("cfg", [dh.SMOLLM2_135M, dh.QWEN3_0_6B], ids=lambda c: c["name"])
def test_decode_after_prefill_matches_a_longer_prefill(torch, cfg):
    from volvoxai_b200 import w8a8
    ctx = w8a8.Context(0)
    ctx.use_torch_stream()
    model = dh.W8A8Decoder(cfg, ctx, w8a8, seed=3, layers=2)
    batch, s = 3, 37
    tokens = torch.randint(0, cfg["vocab"], (batch, s + 1), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    model.allocate_cache(batch, 64)
    want = model.prefill(tokens)                             # positions 0..S, logits at S
    model.allocate_cache(batch, 64, shuffle_seed=7)          # a different scatter of the blocks
    model.prefill(tokens[:, :s])
    pos = torch.full((batch, 1), s, dtype=torch.int64, device="cuda")
    got = model.decode_step(tokens[:, s].contiguous(), pos)
    assert "decode" in w8a8.last_route()
    assert rel(got, want) <= LOGIT_TOL
    # identity block table: the same logits bit for bit (addressing only moves rows)
    model.allocate_cache(batch, 64)
    model.block_table.copy_(torch.arange(model.block_table.numel(), device="cuda").view_as(model.block_table))
    model.prefill(tokens[:, :s])
    again = model.decode_step(tokens[:, s].contiguous(), pos)
    assert torch.equal(again, got)
    model.close()
    ctx.close()


def test_decode_step_replays_from_a_cuda_graph(torch):
    from volvoxai_b200 import w8a8
    cfg = dh.QWEN3_0_6B
    ctx = w8a8.Context(0)
    ctx.use_torch_stream()
    model = dh.W8A8Decoder(cfg, ctx, w8a8, seed=5, layers=2)
    batch, s = 4, 20
    model.allocate_cache(batch, 48)
    prompt = torch.randint(0, cfg["vocab"], (batch, s), device="cuda", generator=torch.Generator(device="cuda").manual_seed(2))
    logits = model.prefill(prompt)
    tok = logits.argmax(-1)
    pos = torch.full((batch, 1), s, dtype=torch.int64, device="cuda")
    eager = []
    k0, v0 = model.k_cache.clone(), model.v_cache.clone()
    t, p = tok.clone(), pos.clone()
    for _ in range(3):
        lg = model.decode_step(t, p)
        eager.append(lg.clone())
        t, p = lg.argmax(-1), p + 1
    model.k_cache.copy_(k0); model.v_cache.copy_(v0)
    t_in, p_in = tok.clone(), pos.clone()
    model.decode_step(t_in, p_in)                            # warm-up outside the capture
    model.k_cache.copy_(k0); model.v_cache.copy_(v0)
    torch.cuda.synchronize()
    side, g = torch.cuda.Stream(), torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        ctx.use_torch_stream()
        out = model.decode_step(t_in, p_in)
    ctx.use_torch_stream()
    for i in range(3):
        g.replay()
        torch.cuda.synchronize()
        assert rel(out, eager[i]) <= 1e-5
        t_in.copy_(out.argmax(-1)); p_in.add_(1)
    model.close()
    ctx.close()
