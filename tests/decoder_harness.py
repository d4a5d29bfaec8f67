"""Decoder harness for the two model-shaped benchmark configurations (measurement and test glue,
not part of the product package).

A Llama-style decoder with random-initialised weights of the configured architecture
(SmolLM2-135M shape: 30 layers, hidden 576, 9 query / 3 KV heads of 64, SwiGLU 1536, vocab 49152;
Qwen3-0.6B shape: 28 layers, hidden 1024, 16 / 8 heads of 128 with per-head q/k RMSNorm, SwiGLU
3072, vocab 151936).  Every q/k/v/o/gate/up/down linear runs through the C ABI of libvxb200.so in
the fused forms the reference's decode path uses (RMSNorm + {q,k,v} sharing one quantization,
RMSNorm + gate/up + SiLU*Mul, o / down projection + residual Add:
native/src/backends/cuda/kernels/cuda_forward_gemv_pair_kernels.inc:155-1711, recognised at
native/src/runtime/incremental_runtime.c:1178-1232).  Everything else is PyTorch glue and is named
as such in the results: embedding lookup, rotary embedding, attention (scaled_dot_product_attention
with grouped KV heads), the paged KV cache (blocks of 16 token slots addressed through per-sequence
block tables, as native/src/runtime/paged_kv.h lays rows out: a token's row is
block_table[pos // 16] * 16 + pos % 16), the final norm and the fp32 lm_head.
"""
from __future__ import annotations

import numpy as np

SMOLLM2_135M = {"name": "smollm2-135m", "layers": 30, "hidden": 576, "heads": 9, "kv_heads": 3, "head_dim": 64,
                "intermediate": 1536, "vocab": 49152, "eps": 1e-5, "qk_norm": False, "rope_theta": 10000.0}
QWEN3_0_6B = {"name": "qwen3-0.6b", "layers": 28, "hidden": 1024, "heads": 16, "kv_heads": 8, "head_dim": 128,
              "intermediate": 3072, "vocab": 151936, "eps": 1e-6, "qk_norm": True, "rope_theta": 1000000.0}
KV_BLOCK = 16


def quantize_per_channel_torch(wf):
    """fp32 [N, K] (device) -> (int8 codes, fp32 scales) with the PTQ packer's arithmetic
    (native/src/training/quantization.c:258-306): scale = absmax / 127 (1 for a zero row),
    codes = ties-to-even(w / scale) clamped to +-127."""
    import torch
    amax = wf.abs().amax(dim=1).double()
    scale = torch.where(amax == 0, torch.ones_like(amax), amax / 127.0).float()
    q = torch.round(wf.double() / scale.double()[:, None]).clamp_(-127, 127).to(torch.int8)
    return q, scale


class W8A8Decoder:
    def __init__(self, cfg: dict, ctx, w8a8, seed: int = 0, layers: int | None = None, device: str = "cuda"):
        import torch
        self.torch, self.cfg, self.ctx, self.w8a8, self.device = torch, dict(cfg), ctx, w8a8, device
        if layers is not None:
            self.cfg["layers"] = layers
        c = self.cfg
        h, hd, nh, nkv, inter = c["hidden"], c["head_dim"], c["heads"], c["kv_heads"], c["intermediate"]
        gen = torch.Generator(device=device).manual_seed(seed)

        def randn(*shape, std=0.02):
            return torch.randn(shape, device=device, generator=gen) * std

        def weight(wf):
            q, s = quantize_per_channel_torch(wf)
            return w8a8.Weight.from_i8(ctx, q.cpu().numpy(), s.cpu().numpy())

        self.embed = randn(c["vocab"], h)
        self.lm_head = randn(c["vocab"], h)
        self.final_norm = torch.ones(h, device=device)
        self.layers = []
        self.weight_bytes = 0
        for _ in range(c["layers"]):
            wq, wk, wv = randn(nh * hd, h), randn(nkv * hd, h), randn(nkv * hd, h)
            gate, up = randn(inter, h), randn(inter, h)
            gate_up = torch.stack([gate, up], dim=1).reshape(2 * inter, h)     # (gate_0, up_0, gate_1, up_1, ...)
            layer = {"qkv": weight(torch.cat([wq, wk, wv], dim=0)), "o": weight(randn(h, nh * hd)),
                     "gate_up": weight(gate_up), "down": weight(randn(h, inter)),
                     "norm1": torch.ones(h, device=device), "norm2": torch.ones(h, device=device)}
            if c["qk_norm"]:
                layer["q_norm"], layer["k_norm"] = torch.ones(hd, device=device), torch.ones(hd, device=device)
            self.layers.append(layer)
            self.weight_bytes += h * (nh + 2 * nkv) * hd + h * nh * hd + 3 * h * inter
        self.k_cache = self.v_cache = self.block_table = None

    # ---- paged KV cache --------------------------------------------------------------------------
    def allocate_cache(self, batch: int, max_len: int, dtype=None, shuffle_seed: int = 1):
        """Blocks of 16 token slots; every sequence owns ceil(max_len / 16) blocks scattered over the
        pool (a seeded permutation), so that consecutive positions of a sequence are not contiguous."""
        torch, c = self.torch, self.cfg
        dtype = dtype or torch.float32
        per_seq = (max_len + KV_BLOCK - 1) // KV_BLOCK
        blocks = batch * per_seq
        perm = np.random.default_rng(shuffle_seed).permutation(blocks).reshape(batch, per_seq)
        self.block_table = torch.from_numpy(perm.astype(np.int64)).to(self.device)
        shape = (c["layers"], blocks * KV_BLOCK, c["kv_heads"], c["head_dim"])
        self.k_cache, self.v_cache = torch.zeros(shape, dtype=dtype, device=self.device), torch.zeros(shape, dtype=dtype, device=self.device)
        self.max_len = per_seq * KV_BLOCK

    def slot_rows(self, positions):
        """positions [B, T] (int64, device) -> rows of the cache [B, T]: block_table[pos // 16] * 16 + pos % 16."""
        blocks = self.torch.gather(self.block_table, 1, positions // KV_BLOCK)
        return blocks * KV_BLOCK + positions % KV_BLOCK

    # ---- pieces ----------------------------------------------------------------------------------
    def _rope(self, x, positions):
        """x [B, T, H, hd], positions [B, T]: rotate-half rotary embedding."""
        torch, c = self.torch, self.cfg
        half = c["head_dim"] // 2
        inv = 1.0 / (c["rope_theta"] ** (torch.arange(half, device=x.device, dtype=torch.float32) / half))
        ang = positions[..., None].float() * inv                      # [B, T, half]
        cos, sin = ang.cos()[:, :, None, :], ang.sin()[:, :, None, :]
        x1, x2 = x[..., :half], x[..., half:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)

    def _head_norm(self, x, w):
        return x * self.torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.cfg["eps"]) * w

    def _layer(self, li, layer, x, positions, batch, t, decode):
        """x [B*T, hidden] fp32 -> [B*T, hidden].  Linears through the library, the rest torch."""
        torch, c, ctx = self.torch, self.cfg, self.ctx
        nh, nkv, hd = c["heads"], c["kv_heads"], c["head_dim"]
        qkv = ctx.rmsnorm_linear_f32_fused(layer["qkv"], x, layer["norm1"], c["eps"])
        q, k, v = qkv.view(batch, t, nh + 2 * nkv, hd).split([nh, nkv, nkv], dim=2)
        if c["qk_norm"]:
            q, k = self._head_norm(q, layer["q_norm"]), self._head_norm(k, layer["k_norm"])
        q, k = self._rope(q, positions), self._rope(k, positions)
        rows = self.slot_rows(positions).reshape(-1)
        self.k_cache[li].index_copy_(0, rows, k.reshape(-1, nkv, hd).to(self.k_cache.dtype))
        self.v_cache[li].index_copy_(0, rows, v.reshape(-1, nkv, hd).to(self.v_cache.dtype))
        if decode:
            # attend over the sequence's cache rows (gathered through its block table), masked beyond its
            # position; the query heads of one KV head ride along as query positions, so K and V are
            # neither expanded nor converted
            all_rows = (self.block_table[:, :, None] * KV_BLOCK + torch.arange(KV_BLOCK, device=x.device)).reshape(batch, -1)
            kk = self.k_cache[li][all_rows].permute(0, 2, 1, 3)          # [B, KV, L, hd]
            vv = self.v_cache[li][all_rows].permute(0, 2, 1, 3)
            qg = q.reshape(batch, nkv, nh // nkv, hd).to(kk.dtype)
            mask = (torch.arange(self.max_len, device=x.device)[None, :] <= positions[:, :1])[:, None, None, :]
            attn = torch.nn.functional.scaled_dot_product_attention(qg, kk, vv, attn_mask=mask).float()
            attn = attn.reshape(batch, nh * hd)                          # head h = kv * group + g, as the query heads were grouped
        else:
            attn = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                                    is_causal=True, enable_gqa=True)
            attn = attn.transpose(1, 2).reshape(batch * t, nh * hd).contiguous()
        x = ctx.linear_f32_fused(layer["o"], attn, residual=x)
        hmid = ctx.rmsnorm_linear_f32_fused(layer["gate_up"], x, layer["norm2"], c["eps"], silu_mul=True)
        return ctx.linear_f32_fused(layer["down"], hmid, residual=x)

    def _logits(self, x_last):
        torch, c = self.torch, self.cfg
        xn = x_last * torch.rsqrt(x_last.pow(2).mean(-1, keepdim=True) + c["eps"]) * self.final_norm
        return xn @ self.lm_head.t()

    # ---- entry points ----------------------------------------------------------------------------
    def prefill(self, tokens):
        """tokens [B, S] int64 -> logits of the last position [B, vocab]; fills the KV cache rows 0..S-1."""
        torch = self.torch
        batch, s = tokens.shape
        positions = torch.arange(s, device=tokens.device)[None, :].expand(batch, s).contiguous()
        x = self.embed[tokens.reshape(-1)]
        for li, layer in enumerate(self.layers):
            x = self._layer(li, layer, x, positions, batch, s, decode=False)
        return self._logits(x.view(batch, s, -1)[:, -1])

    def decode_step(self, tokens, positions):
        """tokens [B], positions [B, 1] (device tensors; static shapes, so the step can be captured in a
        CUDA graph and replayed with updated contents) -> logits [B, vocab]."""
        batch = tokens.shape[0]
        x = self.embed[tokens]
        for li, layer in enumerate(self.layers):
            x = self._layer(li, layer, x, positions, batch, 1, decode=True)
        return self._logits(x)

    def close(self):
        for layer in self.layers:
            for key in ("qkv", "o", "gate_up", "down"):
                layer[key].close()
        self.layers = []
