"""The CPU restatement of the denoise step (oracle/mmdit_oracle.py) runs on its own, at a small
size, and its two attention engines -- the reference's CPU fl_attention and the oracle's float64
restatement -- give the same step. This is the checker the GPU parity test and the benchmark's CPU
baseline use; no GPU and no product kernel is involved."""
import numpy as np
import pytest


def test_cpu_step_runs_and_its_attention_engines_agree(oracle):
    import torch
    from libwaifu_b200.mmdit import MMDiT, MMDiTConfig
    from oracle.mmdit_oracle import OracleBackend
    cfg = MMDiTConfig(hidden=128, heads=2, head_dim=64, mlp=256, blocks=2, text_tokens=8, image_tokens=24, batch=2,
                      latent_channels=16, context_size=48, timestep_embed_dim=32)
    g = torch.Generator().manual_seed(9)
    tokens = torch.randn(cfg.batch, cfg.image_tokens, cfg.latent_channels, generator=g).bfloat16()
    context = torch.randn(cfg.batch, cfg.text_tokens, cfg.context_size, generator=g).bfloat16()
    sinusoid = torch.randn(cfg.batch, cfg.timestep_embed_dim, generator=g).bfloat16()
    engines = ["float64"] + (["reference"] if oracle.have_ref() else [])
    outs = []
    for engine in engines:
        model = MMDiT(cfg, OracleBackend(oracle, attention=engine), seed=0, cpu_init=True)
        with torch.no_grad():
            v = model.step(tokens, context, sinusoid)
        assert v.shape == (cfg.batch, cfg.image_tokens, cfg.latent_channels)
        assert torch.isfinite(v.float()).all() and float(v.float().abs().max()) > 0
        outs.append(v.float().numpy())
    if len(outs) == 2:
        assert oracle.rel_l2(outs[0], outs[1]) <= 2e-2
    # the flop counts the benchmark divides by
    full = MMDiTConfig()
    assert abs(full.gemm_flops() - (118.283e12 + full.outer_gemm_flops())) < 1e10
    assert full.outer_gemm_flops() < 0.001 * full.gemm_flops()
