"""The kernel layer's public names (functional + module wrappers) on CPU: every entry point agrees with the plain
PyTorch formula of the same operation."""
import torch
import torch.nn.functional as F

import trainscale_b200.kernels as K


def test_capability_probe_and_names():
    caps = K.get_kernel_capabilities()
    assert caps["triton"] is False and caps["libraries_built"] is True and not K.is_triton_available()
    assert K.get_accelerator_arch() in set(K.AcceleratorArch)
    for name in ("compile_model", "CompilationConfig", "InductorConfig", "Fast_CrossEntropyLoss", "DistributedKernels",
                 "pinned_memory_transfer", "Fast_RMS_LayerNorm", "Fast_SwiGLU", "Fast_RoPE_Embedding", "FlexAttention",
                 "FP8Linear", "LoRA_MLP", "LoRA_QKV", "moe_grouped_gemm", "torch_amp_custom_fwd"):
        assert hasattr(K, name), name


def test_norms_activations_losses_match_torch():
    torch.manual_seed(0)
    x, r, w, b = torch.randn(6, 64), torch.randn(6, 64), torch.rand(64) + 0.5, torch.randn(64)
    rms = lambda t: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-6) * w      # noqa: E731
    torch.testing.assert_close(K.fast_rms_layernorm(x, w), rms(x))
    y, res = K.fused_add_rms_layernorm(x, r, w, return_residual=True)
    torch.testing.assert_close(res, x + r)
    torch.testing.assert_close(y, rms(x + r))
    torch.testing.assert_close(K.fused_layer_norm(x, w, b), F.layer_norm(x, (64,), w, b))
    torch.testing.assert_close(K.fused_softmax(x), torch.softmax(x, -1))
    torch.testing.assert_close(K.fused_gelu(x), F.gelu(x, approximate="tanh"))
    torch.testing.assert_close(K.swiglu_forward(x, r), F.silu(x) * r)
    torch.testing.assert_close(K.geglu_forward(x, r), F.gelu(x, approximate="tanh") * r)
    logits, labels = torch.randn(2, 5, 11), torch.randint(0, 11, (2, 5))
    labels[0, 0] = -100
    torch.testing.assert_close(K.fast_cross_entropy_loss(logits, labels),
                               F.cross_entropy(logits.view(-1, 11), labels.view(-1), ignore_index=-100))
    assert K.fast_cross_entropy_loss(logits, labels, reduction="none").shape == labels.shape
    assert K.TritonSwiGLU(64, 128)(x).shape == x.shape and K.TritonRMSNorm(64)(x).shape == x.shape


def test_attention_rope_entry_points():
    torch.manual_seed(0)
    q, k, v = torch.randn(2, 16, 4, 16), torch.randn(2, 16, 2, 16), torch.randn(2, 16, 2, 16)
    want = F.scaled_dot_product_attention(q.transpose(1, 2), k.repeat_interleave(2, 2).transpose(1, 2),
                                          v.repeat_interleave(2, 2).transpose(1, 2), is_causal=True).transpose(1, 2)
    torch.testing.assert_close(K.flash_attention(q, k, v), want, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(K.naive_attention(q, k, v), want, rtol=1e-4, atol=1e-5)
    kk, vv = k.repeat_interleave(2, 2), v.repeat_interleave(2, 2)
    torch.testing.assert_close(K.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2),
                                                              is_causal=True).transpose(1, 2), want, rtol=1e-4, atol=1e-5)
    m = K.create_sliding_window_causal_mask(6, 2)
    assert m[3, 2] == 0 and m[3, 3] == 0 and m[3, 1] == float("-inf") and m[2, 3] == float("-inf")
    win = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2),
                                         attn_mask=K.create_sliding_window_causal_mask(16, 4)).transpose(1, 2)
    torch.testing.assert_close(K.flash_attention(q, k, v, window_size=4), win, rtol=1e-4, atol=1e-5)
    capped = K.attention_softcapping_compiled(q, k, v, 5.0)
    torch.testing.assert_close(capped, K.slow_attention_softcapping(q, k, v, 5.0))
    dec = K.inference_attention_single_token(q[:, -1], k, v)
    torch.testing.assert_close(dec, want[:, -1], rtol=1e-4, atol=1e-5)                # last row of causal attention
    cos, sin = K.precompute_freqs_cis(16, 32)
    qr, kr = K.fast_rope_embedding(q, k, cos, sin)
    a, bb = q[..., :8], q[..., 8:]
    c, s = cos[:16, None, :], sin[:16, None, :]
    torch.testing.assert_close(qr, torch.cat((a * c - bb * s, bb * c + a * s), -1), rtol=1e-5, atol=1e-6)
    assert kr.shape == k.shape and K.MultiHeadFlashAttention(64, 4, 2, 16)(torch.randn(2, 16, 64)).shape == (2, 16, 64)
    cache = K.RoPEFrequencyCache()
    cfg = K.RoPEConfig(dim=16, scaling_type=K.RoPEScalingType.YARN, scaling_factor=4.0, max_position=64)
    assert cache.get(cfg, 32)[0].shape == (64, 8) and cache.get(cfg, 32) is cache.get(cfg, 16)


def test_lora_moe_fp8_entry_points():
    torch.manual_seed(0)
    rep = K.validate_lora_gradients()
    assert rep["passed"], rep
    x = torch.randn(8, 64)
    mlp = K.LoRA_MLP(64, 128, r=4)
    assert mlp(x).shape == (8, 64) and not mlp.W_gate.requires_grad and mlp.A_gate.requires_grad
    assert [t.shape[-1] for t in K.LoRA_QKV(64, 64, 32, r=4)(x)] == [64, 32, 32]
    W, A, B = torch.randn(32, 64), torch.randn(4, 64), torch.randn(32, 4)
    torch.testing.assert_close(K.matmul_lora(x, W, A, B, 0.5), x @ W.t() + 0.5 * (x @ A.t()) @ B.t(), rtol=1e-4, atol=1e-4)
    ids, w = torch.randint(0, 4, (8, 2)), torch.softmax(torch.randn(8, 2), -1)
    wgu, wd = torch.randn(4, 64, 64) * 0.1, torch.randn(4, 64, 32) * 0.1
    want = torch.zeros(8, 64)
    for t in range(8):
        for j in range(2):
            g, u = (x[t] @ wgu[ids[t, j]].t()).chunk(2)
            want[t] += w[t, j] * ((F.silu(g) * u) @ wd[ids[t, j]].t())
    torch.testing.assert_close(K.moe_grouped_gemm(x, ids, w, wgu, wd), want, rtol=1e-4, atol=1e-5)
    mgr = K.FP8ScaleManager()
    assert mgr.update("act", torch.tensor([2.0, -4.0])) == 448.0 / 4.0 and mgr.update("act", torch.tensor([1.0])) == 112.0
    assert K.FP8Linear(64, 32, dtype=torch.float32)(x).shape == (8, 32)


def test_longrope_uses_its_factor_lists_and_refuses_to_guess():
    import math

    import pytest
    import torch

    from trainscale_b200.kernels import RoPEConfig, RoPEFrequencyCache, RoPEScalingType
    from trainscale_b200.ops import rope
    half = 32
    lf = [1.0 + 0.1 * i for i in range(half)]
    base = rope.rope_inv_freq(64, 10000.0)
    inv = rope.rope_inv_freq(64, 10000.0, scaling="longrope", original_max_pos=128, max_pos=512, long_factor=lf)
    assert torch.allclose(inv, base / torch.tensor(lf))
    with pytest.raises(ValueError):
        rope.rope_inv_freq(64, 10000.0, scaling="longrope", original_max_pos=128, max_pos=512)
    cfg = RoPEConfig(dim=64, max_position=512, scaling_type=RoPEScalingType.LONGROPE, original_max_position=128,
                     longrope_long_factor=lf)
    cos, _ = RoPEFrequencyCache().get(cfg, 512)
    m = math.sqrt(1 + math.log(4) / math.log(128))
    want = torch.outer(torch.arange(512, dtype=torch.float32), base / torch.tensor(lf)).cos() * m
    assert (cos - want).abs().max() < 1e-3
