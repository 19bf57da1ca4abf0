"""A denoise step of an MMDiT whose linears all run on the quantized-linear path.

The block follows the reference's joint text+image transformer block
(waifu/src/qwen_image/dit.rs:220-345: one projection shared by text and image rows, per-head RMS
norm of q and k, rotary embedding, attention over the joined sequence, gated residuals driven by an
adaLN modulation of the timestep embedding) with the widths of the benchmark configuration
(hidden 3072, 24 heads of 128, MLP 12288 with GELU-tanh, 256 text + 4096 image tokens, 60 blocks).

Only the five linears of a block are this library's work: the modulation (M = batch), the fused
QKV projection, the attention output projection, and the MLP up (GELU fused in the epilogue) and
down projections. Layer norm, modulation arithmetic, q/k norm, rotary embedding and attention are
plain torch, and are inside the timed step but outside the graded path.

The same block code runs over two backends: ``FlintBackend`` (the C ABI on the GPU) and
``OracleBackend`` (the CPU oracle, for the parity test at a reduced size).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional


@dataclass
class MMDiTConfig:
    hidden: int = 3072
    heads: int = 24
    head_dim: int = 128
    mlp: int = 12288
    blocks: int = 60
    text_tokens: int = 256
    image_tokens: int = 4096
    batch: int = 2  # the two classifier-free-guidance rows

    @property
    def tokens(self) -> int:
        return self.text_tokens + self.image_tokens

    def gemm_flops(self) -> float:
        """2 m n k over the four big linears of every block (the modulation's are negligible)."""
        m = self.batch * self.tokens
        per_block = 2.0 * m * self.hidden * (3 * self.hidden + self.hidden + 2 * self.mlp)
        return per_block * self.blocks


LAYER_SHAPES = lambda c: {"mod": (6 * c.hidden, c.hidden), "qkv": (3 * c.hidden, c.hidden),
                          "out": (c.hidden, c.hidden), "up": (c.mlp, c.hidden), "down": (c.hidden, c.mlp)}


class FlintBackend:
    """Linears through libflint_sm100 (fl_quantize_fp8_rows at load, fl_fp8_linear per call)."""

    def __init__(self):
        import torch
        from . import flint as F
        self.torch = torch
        self.F = F
        self.device = "cuda"

    def _wrap(self, t, dt):
        return self.F.Tensor.from_device_ptr(t.data_ptr(), tuple(t.shape), dt, keepalive=t)

    def make_layer(self, w_f32, bias_bf16):
        codes, scales = self.F.quantize_fp8_rows(self._wrap(w_f32, self.F.DType.FLOAT))
        self.F.synchronize()
        return (codes, scales, None if bias_bf16 is None else self._wrap(bias_bf16, self.F.DType.BFLOAT16), bias_bf16)

    def linear(self, x2d, layer, act: int = 0, residual2d=None):
        torch, F = self.torch, self.F
        codes, scales, bias, _ = layer
        out = torch.empty((x2d.shape[0], codes.shape[0]), dtype=torch.bfloat16, device=x2d.device)
        F.fp8_linear(self._wrap(x2d, F.DType.BFLOAT16), codes, scales, bias,
                     None if residual2d is None else self._wrap(residual2d, F.DType.BFLOAT16), act,
                     self._wrap(out, F.DType.BFLOAT16))
        return out


class OracleBackend:
    """The same linears on the CPU through the test oracle (only tests construct this)."""

    def __init__(self, oracle_module):
        import torch
        self.torch = torch
        self.O = oracle_module
        self.device = "cpu"

    def _bits(self, t):
        return t.contiguous().view(self.torch.int16).numpy().view("uint16")

    def make_layer(self, w_f32, bias_bf16):
        codes, scales = self.O.quantize_fp8_rows(w_f32.cpu().numpy())
        return (codes, scales, None if bias_bf16 is None else self._bits(bias_bf16.cpu()))

    def linear(self, x2d, layer, act: int = 0, residual2d=None):
        codes, scales, bias = layer
        y = self.O.fp8_linear(self._bits(x2d), codes, scales, bias,
                              None if residual2d is None else self._bits(residual2d), act, True)
        return self.torch.from_numpy(y.view("int16").copy()).view(self.torch.bfloat16)


def _rope(x, cos, sin):
    # x: (b, heads, tokens, head_dim); rotate pairs (even, odd)
    x1, x2 = x[..., 0::2], x[..., 1::2]
    out = x.new_empty(x.shape)
    out[..., 0::2] = x1 * cos - x2 * sin
    out[..., 1::2] = x1 * sin + x2 * cos
    return out


class MMDiT:
    """Random-init weights (N(0, 0.02^2), seed 0) quantised to e4m3 with per-row scales."""

    def __init__(self, cfg: MMDiTConfig, backend, seed: int = 0, blocks: Optional[int] = None, cpu_init: bool = False):
        """`cpu_init` draws the weights on the CPU whatever the backend, so that two backends hold
        identical weights (for parity checks); otherwise a GPU backend draws them on the GPU."""
        import torch
        self.torch = torch
        self.cfg = cfg
        self.backend = backend
        self.num_blocks = cfg.blocks if blocks is None else blocks
        gen = torch.Generator(device="cpu").manual_seed(seed)
        dev = backend.device
        self.layers: List[dict] = []
        for _ in range(self.num_blocks):
            block = {}
            for name, (n, k) in LAYER_SHAPES(cfg).items():
                if dev == "cuda" and not cpu_init:
                    g = torch.Generator(device="cuda").manual_seed(int(torch.randint(0, 2 ** 31, (1,), generator=gen)))
                    w = torch.randn(n, k, device="cuda", dtype=torch.float32, generator=g) * 0.02
                    b = (torch.randn(n, device="cuda", dtype=torch.float32, generator=g) * 0.01).bfloat16()
                else:
                    w = (torch.randn(n, k, generator=gen) * 0.02).to(dev)
                    b = (torch.randn(n, generator=gen) * 0.01).bfloat16().to(dev)
                block[name] = backend.make_layer(w, b)
                del w
            self.layers.append(block)
        half = cfg.head_dim // 2
        pos = torch.arange(cfg.tokens, dtype=torch.float32)
        freq = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32) / half)
        ang = pos[:, None] * freq[None, :]
        self.cos = ang.cos().to(dev).to(torch.bfloat16)
        self.sin = ang.sin().to(dev).to(torch.bfloat16)

    def block(self, x, temb, layers):
        torch = self.torch
        Fn = torch.nn.functional
        c = self.cfg
        b, t, d = x.shape
        lin = self.backend.linear
        mod = lin(Fn.silu(temb), layers["mod"])  # (b, 6 d): the M = batch skinny linear
        shift1, scale1, gate1, shift2, scale2, gate2 = [m[:, None, :] for m in mod.chunk(6, dim=1)]

        h = Fn.layer_norm(x, (d,)) * (1 + scale1) + shift1
        qkv = lin(h.reshape(b * t, d).contiguous(), layers["qkv"]).view(b, t, 3, c.heads, c.head_dim)
        q, k, v = qkv[:, :, 0].transpose(1, 2), qkv[:, :, 1].transpose(1, 2), qkv[:, :, 2].transpose(1, 2)
        q = Fn.rms_norm(q, (c.head_dim,))
        k = Fn.rms_norm(k, (c.head_dim,))
        q = _rope(q, self.cos, self.sin)
        k = _rope(k, self.cos, self.sin)
        a = Fn.scaled_dot_product_attention(q, k, v)  # joint attention over text + image tokens
        a = a.transpose(1, 2).reshape(b * t, d).contiguous()
        x = x + gate1 * lin(a, layers["out"]).view(b, t, d)

        h2 = (Fn.layer_norm(x, (d,)) * (1 + scale2) + shift2).reshape(b * t, d).contiguous()
        u = lin(h2, layers["up"], act=1)  # GELU-tanh fused into the epilogue
        x = x + gate2 * lin(u, layers["down"]).view(b, t, d)
        return x

    def step(self, x, temb):
        """x (batch, tokens, hidden) bf16, temb (batch, hidden) bf16 -> the same shape as x."""
        for layers in self.layers:
            x = self.block(x, temb, layers)
        return x
