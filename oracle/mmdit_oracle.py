"""Test infrastructure, not product code: the CPU side of the denoise step.

``OracleBackend`` offers the methods ``libwaifu_b200.mmdit.MMDiT`` asks of a backend, each fused
step of the GPU path spelled out as the separate operations it stands for, all on the host: the
linears through the oracle's restated quantisers with the float32 product taken by the reference's
own CPU ``fl_matmul`` where it was built (oracle/_ref), the attention through the reference's own
CPU ``fl_attention`` (float32, flint/operators.cc:148-230), the rest in numpy float32 in the
reference's operation order. Only the parity tests and ``bench.py``'s CPU-baseline leg construct it.
"""
from __future__ import annotations

import numpy as np

LN_EPS = 1e-6


class OracleBackend:
    def __init__(self, oracle_module, attention: str = "auto"):
        """`attention`: "reference" (the reference's CPU fl_attention), "float64" (the oracle's own
        restatement), or "auto": the first where the reference's library was built, else the second."""
        import torch
        self.torch = torch
        self.O = oracle_module
        self.device = "cpu"
        if attention == "auto":
            attention = "reference" if oracle_module.have_ref() else "float64"
        self.attention_engine = attention

    def _bits(self, t):
        return t.contiguous().view(self.torch.int16).numpy().view("uint16")

    def _tensor(self, bits):
        return self.torch.from_numpy(np.ascontiguousarray(bits).view("int16").copy()).view(self.torch.bfloat16)

    def make_layer(self, w_f32, bias_bf16):
        codes, scales = self.O.quantize_fp8_rows(w_f32.cpu().numpy())
        return (codes, scales, None if bias_bf16 is None else self._bits(bias_bf16.cpu()))

    def linear(self, x2d, layer, act: int = 0, residual2d=None):
        codes, scales, bias = layer
        y = self.O.fp8_linear(self._bits(x2d), codes, scales, bias,
                              None if residual2d is None else self._bits(residual2d), act, True)
        return self._tensor(y)

    def silu(self, x):
        return self.torch.nn.functional.silu(x)

    def rms_norm(self, x2d, weight_f32, eps):
        a = x2d.float().numpy()
        w = weight_f32.numpy().astype(np.float32)
        ms = (a.astype(np.float64) ** 2).mean(axis=1, keepdims=True).astype(np.float32)
        y = (a * w / np.sqrt(ms + np.float32(eps), dtype=np.float32)).astype(np.float32)
        return self._tensor(self.O.narrow(y, True))

    def modulated_linear(self, x3d, scale, shift, layer, act: int = 0):
        b, t, d = x3d.shape
        h = self.O.layernorm_modulate(self._bits(x3d.reshape(b * t, d)), self._bits(scale),
                                      None if shift is None else self._bits(shift), LN_EPS, True)
        return self.linear(self._tensor(h), layer, act)

    def qk_norm_rope(self, qkv2d, cos, sin, heads):
        return self._tensor(self.O.qk_norm_rope(self._bits(qkv2d), cos.numpy(), sin.numpy(), heads, LN_EPS, True))

    def attention(self, qkv5d):
        torch = self.torch
        b, t, _, h, hd = qkv5d.shape
        q, k, v = (qkv5d[:, :, i].transpose(1, 2).contiguous() for i in range(3))  # (b, h, t, hd)
        if self.attention_engine == "reference":
            a = self.O.ref().attention(q.float().numpy(), k.float().numpy(), v.float().numpy(), False)
        else:
            a = self.O.attention(self._bits(q), self._bits(k), self._bits(v), False, True).astype(np.float32)
        a = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16)
        return a.transpose(1, 2).reshape(b * t, h * hd).contiguous()

    def gated_linear(self, a2d, layer, gate, stream3d):
        b, t, n = stream3d.shape
        y = self.linear(a2d, layer).view(b, t, n).float()
        return (stream3d.float() + gate[:, None, :].float() * y).to(self.torch.bfloat16)
