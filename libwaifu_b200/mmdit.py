"""A denoise step of an MMDiT whose linears all run on the quantized-linear path.

The step follows the reference's denoiser (waifu/src/qwen_image/dit.rs:448-578): the timestep's
sinusoid goes through the two time-embed linears (M = batch rows), the prompt's encoder states
through an RMS norm and the two `txt_in` linears, the latent tokens through `img_in` (64 -> hidden),
text and image rows are joined (prompt first) and walked through the blocks, and the last layer
reads the picture's rows only: a scale off the step's own embedding, layer norm times (1 + scale),
and the projection back to the latent's 64 channels.

The block follows the reference's joint text+image transformer block
(waifu/src/qwen_image/dit.rs:220-345: one projection shared by text and image rows, per-head RMS
norm of q and k, rotary embedding, attention over the joined sequence, gated residuals driven by an
adaLN modulation of the timestep embedding) with the widths of the benchmark configuration
(hidden 3072, 24 heads of 128, MLP 12288 with GELU-tanh, 256 text + 4096 image tokens, 60 blocks).

The five linears of a block are this library's work: the modulation (M = batch), the fused QKV
projection, the attention output projection, and the MLP up (GELU fused in the epilogue) and down
projections, together with the steps either side of them: layer norm, adaLN modulation and the
activation quantiser run as one kernel in front of the QKV and up projections
(fl_fp8_layernorm_quantize), and the gated residual `x + gate * linear(a)` behind the output and
down projections is folded into the projection's epilogue (the gate multiplies the per-channel
scale and the bias, the stream is the residual), and the per-head RMS norm of q and k with their
rotary embedding runs in place on the QKV projection's output (fl_qk_norm_rope), which attention
then reads as three strided views. Attention runs through this library's fl_attention by default
(the same strided views, the result written token-major); ``FlintBackend(attention_kernel="sdpa")``
swaps in torch's scaled_dot_product_attention, a library kernel kept as a yardstick. The SiLU of
the embeddings and the RMS norm of the prompt's states (0.3 % of a step's rows) are plain torch.

The block code runs over any backend with FlintBackend's methods; the CPU restatement the parity
tests and the CPU baseline use lives with the oracle, outside this package.
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
    latent_channels: int = 64      # a 2 x 2 patch of the 16-channel latent
    context_size: int = 3584       # width of the prompt encoder's states
    timestep_embed_dim: int = 256

    @property
    def tokens(self) -> int:
        return self.text_tokens + self.image_tokens

    def block_gemm_flops(self) -> float:
        """2 m n k over the four big linears of one block (the modulation's are negligible)."""
        m = self.batch * self.tokens
        return 2.0 * m * self.hidden * (3 * self.hidden + self.hidden + 2 * self.mlp)

    def outer_gemm_flops(self) -> float:
        """The linears outside the blocks: txt_in (two), img_in and the final projection."""
        mt, mi, d = self.batch * self.text_tokens, self.batch * self.image_tokens, self.hidden
        return 2.0 * (mt * d * (self.context_size + d) + 2 * mi * d * self.latent_channels)

    def gemm_flops(self, blocks: Optional[int] = None) -> float:
        return self.block_gemm_flops() * (self.blocks if blocks is None else blocks) + self.outer_gemm_flops()

    def attention_flops(self, blocks: Optional[int] = None) -> float:
        per_block = 4.0 * self.batch * self.heads * self.tokens * self.tokens * self.head_dim
        return per_block * (self.blocks if blocks is None else blocks)


LAYER_SHAPES = lambda c: {"mod": (6 * c.hidden, c.hidden), "qkv": (3 * c.hidden, c.hidden),
                          "out": (c.hidden, c.hidden), "up": (c.mlp, c.hidden), "down": (c.hidden, c.mlp)}

# The linears around the blocks (waifu/src/qwen_image/dit.rs:464-475,497-512,565-578), (n, k).
OUTER_SHAPES = lambda c: {"time1": (c.hidden, c.timestep_embed_dim), "time2": (c.hidden, c.hidden),
                          "txt1": (c.hidden, c.context_size), "txt2": (c.hidden, c.hidden),
                          "img_in": (c.hidden, c.latent_channels),
                          "final_lin": (c.hidden, c.hidden), "final_proj": (c.latent_channels, c.hidden)}


LN_EPS = 1e-6


class FlintBackend:
    """Linears through libflint_sm100 (fl_quantize_fp8_rows at load; per call fl_fp8_linear, or
    fl_fp8_layernorm_quantize + fl_fp8_linear_quantized where a layer norm feeds the linear)."""

    def __init__(self, attention_kernel: str = "flint"):
        import torch
        from . import flint as F
        if attention_kernel not in ("sdpa", "flint"):
            raise ValueError("attention_kernel is 'sdpa' or 'flint'")
        self.torch = torch
        self.F = F
        self.device = "cuda"
        self.attention_kernel = attention_kernel

    def _wrap(self, t, dt):
        """A view of a torch tensor's memory with its own strides (a column slice stays a slice)."""
        return self.F.Tensor.from_device_ptr(t.data_ptr(), tuple(t.shape), dt, keepalive=t, stride=tuple(t.stride()),
                                             numel=(t.shape[0] - 1) * t.stride(0) + t.shape[-1] if t.dim() == 2 and not t.is_contiguous() else None)

    def make_layer(self, w_f32, bias_bf16):
        torch, F = self.torch, self.F
        n, k = w_f32.shape
        codes_t = torch.empty((n, k), dtype=torch.uint8, device="cuda")
        scales_t = torch.empty((n,), dtype=torch.float32, device="cuda")
        codes, scales = self._wrap(codes_t, F.DType.FP8E4M3), self._wrap(scales_t, F.DType.FLOAT)
        w = self._wrap(w_f32, F.DType.FLOAT)
        F.check(F.lib().fl_quantize_fp8_rows(w.raw(), codes.raw(), scales.raw()))
        F.synchronize()
        return (codes, scales, None if bias_bf16 is None else self._wrap(bias_bf16, F.DType.BFLOAT16),
                None if bias_bf16 is None else bias_bf16.float(), scales_t)

    def linear(self, x2d, layer, act: int = 0, residual2d=None):
        torch, F = self.torch, self.F
        codes, scales, bias = layer[:3]
        out = torch.empty((x2d.shape[0], codes.shape[0]), dtype=torch.bfloat16, device=x2d.device)
        F.fp8_linear(self._wrap(x2d, F.DType.BFLOAT16), codes, scales, bias,
                     None if residual2d is None else self._wrap(residual2d, F.DType.BFLOAT16), act,
                     self._wrap(out, F.DType.BFLOAT16))
        return out

    def modulated_linear(self, x3d, scale, shift, layer, act: int = 0):
        """linear(round16(LN(x) * scale + LN(x) + shift)) with scale, shift (batch, hidden): one
        kernel reads x and writes the e4m3 rows, the GEMM takes them as they are."""
        torch, F = self.torch, self.F
        codes, scales, bias = layer[:3]
        b, t, d = x3d.shape
        q = torch.empty((b * t, d), dtype=torch.uint8, device=x3d.device)
        rs = torch.empty((b * t,), dtype=torch.float32, device=x3d.device)
        qw, rsw = self._wrap(q, F.DType.FP8E4M3), self._wrap(rs, F.DType.FLOAT)
        # scale and shift are column slices of the modulation linear's output: passed as they lie
        F.fp8_layernorm_quantize(self._wrap(x3d.reshape(b * t, d), F.DType.BFLOAT16), self._wrap(scale, F.DType.BFLOAT16),
                                 None if shift is None else self._wrap(shift, F.DType.BFLOAT16), LN_EPS, qw, rsw)
        out = torch.empty((b * t, codes.shape[0]), dtype=torch.bfloat16, device=x3d.device)
        F.fp8_linear_quantized(qw, rsw, codes, scales, bias, None, act, self._wrap(out, F.DType.BFLOAT16))
        return out

    def silu(self, x):
        return self.torch.nn.functional.silu(x)

    def rms_norm(self, x2d, weight_f32, eps):
        """flint's rmsNorm in float32 (a * w / sqrt(mean(a^2) + eps), flint/cpu/normalizations.cc:33-70),
        narrowed once: the prompt's way in (waifu/src/qwen_image/dit.rs:481-495)."""
        torch = self.torch
        a = x2d.float()
        return (a * weight_f32 / torch.sqrt(a.pow(2).mean(dim=1, keepdim=True) + eps)).to(torch.bfloat16)

    def qk_norm_rope(self, qkv2d, cos, sin, heads):
        """In place: per-head RMS norm of q and k, then their rotary embedding."""
        F = self.F
        F.qk_norm_rope(self._wrap(qkv2d, F.DType.BFLOAT16), self._wrap(cos, F.DType.FLOAT), self._wrap(sin, F.DType.FLOAT),
                       heads, LN_EPS)
        return qkv2d

    def attention(self, qkv5d):
        """Joint attention over qkv (batch, tokens, 3, heads, head_dim), the fused projection's
        output: q, k and v are strided views of it and the result is token-major (batch * tokens,
        heads * head_dim), the layout the next projection reads. `self.attention_kernel` chooses
        this library's kernel ("flint", the default) or torch's ("sdpa", a yardstick)."""
        torch, F = self.torch, self.F
        b, t, _, h, hd = qkv5d.shape
        if self.attention_kernel == "flint":
            out = torch.empty((b, t, h, hd), dtype=torch.bfloat16, device=qkv5d.device)
            views = []
            for i in range(3):
                part = qkv5d[:, :, i].transpose(1, 2)  # (b, h, t, hd)
                views.append(F.Tensor.from_device_ptr(part.data_ptr(), tuple(part.shape), F.DType.BFLOAT16, keepalive=qkv5d,
                                                      stride=tuple(part.stride()), numel=qkv5d.numel()))
            o = out.transpose(1, 2)
            ov = F.Tensor.from_device_ptr(o.data_ptr(), tuple(o.shape), F.DType.BFLOAT16, keepalive=out,
                                          stride=tuple(o.stride()), numel=out.numel())
            F.attention(views[0], views[1], views[2], F.MaskType.NONE, 0, ov)
            return out.view(b * t, h * hd)
        q, k, v = (qkv5d[:, :, i].transpose(1, 2) for i in range(3))
        a = torch.nn.functional.scaled_dot_product_attention(q, k, v)
        a = a.transpose(1, 2).reshape(b * t, h * hd)
        return a if a.is_contiguous() else a.contiguous()

    def gated_linear(self, a2d, layer, gate, stream3d):
        """stream + gate * linear(a), gate (batch, n): per batch row block one GEMM whose per-channel
        scale and bias carry the gate and whose residual is the stream, so the product is rounded
        once and no elementwise pass follows it."""
        torch, F = self.torch, self.F
        codes, scales, bias, bias_f32, scales_t = layer
        b, t, n = stream3d.shape
        out = torch.empty((b, t, n), dtype=torch.bfloat16, device=a2d.device)
        g32 = gate if gate.dtype == torch.float32 else gate.float()
        gated_scales = torch.mul(g32, scales_t)                                      # (b, n) fp32, contiguous
        gated_bias = None if bias_f32 is None else torch.mul(g32, bias_f32).to(torch.bfloat16)
        k = a2d.shape[1]
        q = torch.empty((b * t, k), dtype=torch.uint8, device=a2d.device)
        rs = torch.empty((b * t,), dtype=torch.float32, device=a2d.device)
        aw, qw, rsw = self._wrap(a2d, F.DType.BFLOAT16), self._wrap(q, F.DType.FP8E4M3), self._wrap(rs, F.DType.FLOAT)
        F.check(F.lib().fl_quantize_fp8_activation(aw.raw(), qw.raw(), rsw.raw()))  # the views outlive the call
        if t % 256 == 0:
            # every image's rows are whole tiles of the product: one GEMM whose epilogue takes the
            # scales and the bias of a row's image
            F.fp8_linear_quantized_grouped(qw, rsw, codes, self._wrap(gated_scales, F.DType.FLOAT),
                                           None if gated_bias is None else self._wrap(gated_bias, F.DType.BFLOAT16),
                                           self._wrap(stream3d.reshape(b * t, n), F.DType.BFLOAT16), 0, t,
                                           self._wrap(out.view(b * t, n), F.DType.BFLOAT16))
            return out
        for i in range(b):
            rows = slice(i * t, (i + 1) * t)
            F.fp8_linear_quantized(self._wrap(q[rows], F.DType.FP8E4M3), self._wrap(rs[rows], F.DType.FLOAT), codes,
                                   self._wrap(gated_scales[i], F.DType.FLOAT),
                                   None if gated_bias is None else self._wrap(gated_bias[i], F.DType.BFLOAT16),
                                   self._wrap(stream3d[i], F.DType.BFLOAT16), 0, self._wrap(out[i], F.DType.BFLOAT16))
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
        self.outer = {}
        for name, (n, k) in OUTER_SHAPES(cfg).items():
            if dev == "cuda" and not cpu_init:
                g = torch.Generator(device="cuda").manual_seed(int(torch.randint(0, 2 ** 31, (1,), generator=gen)))
                w = torch.randn(n, k, device="cuda", dtype=torch.float32, generator=g) * 0.02
                b = (torch.randn(n, device="cuda", dtype=torch.float32, generator=g) * 0.01).bfloat16()
            else:
                w = (torch.randn(n, k, generator=gen) * 0.02).to(dev)
                b = (torch.randn(n, generator=gen) * 0.01).bfloat16().to(dev)
            self.outer[name] = backend.make_layer(w, b)
            del w
        self.txt_norm = (1.0 + 0.1 * torch.randn(cfg.context_size, generator=gen)).to(dev)  # float32, as the reference keeps it
        half = cfg.head_dim // 2
        pos = torch.arange(cfg.tokens, dtype=torch.float32)
        freq = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32) / half)
        ang = pos[:, None] * freq[None, :]
        self.cos = ang.cos().contiguous().to(dev)  # float32 (tokens, head_dim / 2)
        self.sin = ang.sin().contiguous().to(dev)

    def block(self, x, temb, layers, tap=None):
        """One block. `tap(name, tensor) -> tensor`, when given, sees every intermediate in turn
        (mod, qkv, qk, attention, x1, up, x2) and what it returns is used in its place: a test
        records one backend's intermediates with it and feeds them to the other backend, so that
        each stage of the two is compared on identical inputs."""
        c = self.cfg
        b, t, d = x.shape
        lin = self.backend.linear
        see = tap if tap is not None else (lambda name, value: value)
        mod = see("mod", lin(self.backend.silu(temb), layers["mod"]))  # (b, 6 d): the M = batch skinny linear
        shift1, scale1, _, shift2, scale2, _ = mod.chunk(6, dim=1)   # column slices, not copies
        modf = mod.float()                                             # the gates multiply fp32 scales
        gate1, gate2 = modf[:, 2 * d:3 * d], modf[:, 5 * d:6 * d]

        qkv = see("qkv", self.backend.modulated_linear(x, scale1, shift1, layers["qkv"]))  # (b t, 3 d)
        qkv = see("qk", self.backend.qk_norm_rope(qkv, self.cos, self.sin, c.heads)).view(b, t, 3, c.heads, c.head_dim)
        # q, k, v as (b, heads, t, head_dim) views of the one buffer: nothing is copied, and the
        # attention output comes back token-major, which is the layout the next projection reads
        a = see("attention", self.backend.attention(qkv))  # joint attention over text + image tokens
        x = see("x1", self.backend.gated_linear(a, layers["out"], gate1, x))

        u = see("up", self.backend.modulated_linear(x, scale2, shift2, layers["up"], act=1))  # GELU-tanh in the epilogue
        x = see("x2", self.backend.gated_linear(u, layers["down"], gate2, x))
        return x

    def embed(self, tokens, context, sinusoid):
        """The ways in (waifu/src/qwen_image/dit.rs:464-512): tokens (batch, image_tokens,
        latent_channels), context (batch, text_tokens, context_size) and sinusoid (batch,
        timestep_embed_dim), all 16-bit -> the joined stream (batch, tokens, hidden), prompt rows
        first, and the timestep embedding (batch, hidden)."""
        torch, c, be = self.torch, self.cfg, self.backend
        lin = be.linear
        b = tokens.shape[0]
        emb = lin(be.silu(lin(sinusoid, self.outer["time1"])), self.outer["time2"])
        normed = be.rms_norm(context.reshape(b * c.text_tokens, c.context_size), self.txt_norm, LN_EPS)
        text = lin(lin(normed, self.outer["txt1"], act=1), self.outer["txt2"])  # GELU-tanh between, in the epilogue
        image = lin(tokens.reshape(b * c.image_tokens, c.latent_channels), self.outer["img_in"])
        x = torch.cat([text.view(b, c.text_tokens, c.hidden), image.view(b, c.image_tokens, c.hidden)], dim=1)
        return x, emb

    def final(self, x, emb):
        """The last layer (waifu/src/qwen_image/dit.rs:565-578) on the picture's rows only: a scale
        off the step's embedding, layer norm times (1 + scale), the projection to the latent."""
        c, be = self.cfg, self.backend
        b = x.shape[0]
        scale = be.linear(be.silu(emb), self.outer["final_lin"])  # (batch, hidden)
        image = x[:, c.text_tokens:].contiguous()
        v = be.modulated_linear(image, scale, None, self.outer["final_proj"])
        return v.view(b, c.image_tokens, c.latent_channels)

    def blocks(self, x, temb):
        """x (batch, tokens, hidden) bf16, temb (batch, hidden) bf16 -> the same shape as x."""
        for layers in self.layers:
            x = self.block(x, temb, layers)
        return x

    def step(self, tokens, context, sinusoid):
        """One denoise step: latent tokens, prompt states and the timestep's sinusoid in, the
        velocity (batch, image_tokens, latent_channels) out."""
        x, emb = self.embed(tokens, context, sinusoid)
        return self.final(self.blocks(x, emb), emb)
