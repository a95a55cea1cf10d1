"""The flex-style attention front end (kernels/flex.py) against direct softmax(QK^T)V math; on CPU every path runs the
fp32 reference of the flash kernels, so this checks the mask / scale / soft-cap / GQA plumbing."""
import math

import torch

from trainscale_b200 import kernels as K


def _direct(Q, Kt, V, allow, scale, softcap=0.0):
    g = Q.shape[1] // Kt.shape[1]
    Kt, V = Kt.repeat_interleave(g, 1), V.repeat_interleave(g, 1)
    s = (Q.float() @ Kt.float().transpose(-1, -2)) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    s = s.masked_fill(~allow, float("-inf"))
    return torch.softmax(s, -1) @ V.float()


def _merge(o):
    return o.transpose(1, 2).reshape(o.shape[0], o.shape[2], -1)


def test_block_masks_are_recognised_and_forwards_match_direct_math():
    torch.manual_seed(0)
    B, H, Hkv, S, D = 2, 4, 2, 24, 16
    Q, Kt, V = torch.randn(B, H, S, D), torch.randn(B, Hkv, S, D), torch.randn(B, Hkv, S, D)
    i = torch.arange(S)
    causal = i[:, None] >= i[None, :]
    cfg = K.FlexAttentionConfig(num_attention_heads=H, num_key_value_heads=Hkv, head_dim=D,
                                attn_logit_softcapping=5.0, query_pre_attn_scalar=float(D))
    assert cfg.num_kv_groups == 2 and cfg.hidden_size == H * D and cfg.softcap == 5.0
    scale = 1 / math.sqrt(D)

    bm = K.create_flex_attention_causal_mask(S)
    assert bm.kind == "causal"
    out = K.flex_attention_forward(Q, Kt, V, bm, cfg)
    assert out.shape == (B, S, H * D)
    assert torch.allclose(out, _merge(_direct(Q, Kt, V, causal, scale, 5.0)), atol=2e-5)

    sw = K.create_flex_attention_sliding_window_mask(S, sliding_window=5)
    assert sw.kind == "sliding_window" and sw.window == 5
    win = causal & (i[:, None] - i[None, :] < 5)
    assert torch.equal(sw.to_bool(), win)
    assert torch.allclose(K.flex_attention_forward(Q, Kt, V, sw, cfg), _merge(_direct(Q, Kt, V, win, scale, 5.0)),
                          atol=2e-5)

    # a hand-written function for ints is evaluated pair by pair; a causal one is recognised by value
    assert K.create_block_mask(lambda b, h, q, k: q >= k and True, 8).kind == "causal"
    odd = K.create_block_mask(lambda b, h, q, k: (q >= k) and ((q - k) % 2 == 0), S)
    assert odd.kind == "dense"
    allow = causal & ((i[:, None] - i[None, :]) % 2 == 0)
    assert torch.allclose(K.flex_attention_forward(Q, Kt, V, odd, cfg), _merge(_direct(Q, Kt, V, allow, scale, 5.0)),
                          atol=2e-5)
    per_head = K.CausalSlidingWindowMasker({0: 3}, default_window=7)
    assert K.create_block_mask(per_head, S, num_heads=H).dense.shape == (H, S, S)
    assert K.create_block_mask(K.CausalSlidingWindowMasker(default_window=7), S, num_heads=H).kind == "sliding_window"

    plain = K.FlexAttentionConfig(num_attention_heads=H, num_key_value_heads=Hkv, head_dim=D)
    assert torch.allclose(K.flash_attention_forward(Q, Kt, V, plain, causal=True), _merge(_direct(Q, Kt, V, causal, scale)),
                          atol=2e-5)
    full = torch.ones(S, S, dtype=torch.bool)
    assert torch.allclose(K.sdpa_attention_forward(Q, Kt, V, plain, is_causal=False), _merge(_direct(Q, Kt, V, full, scale)),
                          atol=2e-5)
    add = torch.zeros(S, S).masked_fill(~win, float("-inf"))
    assert torch.allclose(K.sdpa_attention_forward(Q, Kt, V, plain, attn_mask=add), _merge(_direct(Q, Kt, V, win, scale)),
                          atol=2e-5)
    # no block mask = full attention, as with torch's flex_attention
    fn = K.get_flex_attention(float(D), 0.0)
    assert torch.allclose(fn(Q, Kt, V), _direct(Q, Kt, V, full, scale), atol=2e-5)


def test_generation_step_variants_and_modifiers():
    torch.manual_seed(1)
    B, H, Hkv, S, D = 1, 4, 1, 12, 8
    Kt, V = torch.randn(B, Hkv, S, D), torch.randn(B, Hkv, S, D)
    q1 = torch.randn(B, H, 1, D)
    cfg = K.FlexAttentionConfig(num_attention_heads=H, num_key_value_heads=Hkv, head_dim=D, attn_logit_softcapping=3.0)
    mask = torch.zeros(1, S)                     # the single new token sees the whole cache
    got = K.inference_attention_softcapping(q1, Kt, V, mask, cfg)
    want = _merge(_direct(q1, Kt, V, torch.ones(1, S, dtype=torch.bool), 1 / math.sqrt(D), 3.0))
    assert got.shape == (B, 1, H * D) and torch.allclose(got, want, atol=2e-5)
    assert torch.allclose(K.slow_inference_attention_softcapping(q1, Kt, V, mask, cfg, B, 1), want, atol=2e-5)
    assert torch.allclose(K.attention_sliding_window_compiled(q1, Kt, V, mask, 1.0, 3.0, H, Hkv, D), want, atol=2e-5)
    # a decode step through the flex callable: causal block mask, one query against S keys
    fn = K.get_flex_attention(1.0, 3.0)
    assert torch.allclose(_merge(fn(q1, Kt, V, K.create_flex_attention_causal_mask(S))), want, atol=2e-5)

    s = torch.randn(4, 4) * 10
    assert torch.allclose(K.apply_softcap_stable(s, 2.0), 2 * torch.tanh(s / 2))
    assert torch.allclose(K.apply_softcap_inplace(s.clone(), 2.0), 2 * torch.tanh(s / 2))
    assert torch.allclose(K.generate_tanh_softcap(2.0)(s, 0, 0, 0, 0), 2 * torch.tanh(s / 2), atol=1e-4)
    assert torch.allclose(K.generate_combined_modifier(0.5, 2.0)(s, 0, 0, 0, 0), 2 * torch.tanh(s / 4), atol=1e-4)
    assert torch.equal(K.generate_scale_modifier(0.5)(s, 0, 0, 0, 0), s * 0.5)
    k2, v2 = K.expand_kv_for_gqa_contiguous(Kt, V, 4)
    assert k2.shape == (B, 4, S, D) and k2.is_contiguous() and torch.equal(k2[:, 3], Kt[:, 0])
    assert K.get_causal_mask_slice(torch.ones(8, 8), 2, 5).shape == (2, 5)
    assert K.causal_masker(0, 0, 3, 2) and not K.get_sliding_window_masker(2)(0, 0, 5, 2)


def test_moe_block_router_and_grouped_gemm_functionals():
    import torch.nn.functional as F
    torch.manual_seed(2)
    H, I, E, k = 32, 48, 4, 2
    blk = K.create_moe_block(H, I, num_experts=E, top_k=k).eval()
    x = torch.randn(2, 9, H)
    out, aux = blk(x)
    assert out.shape == x.shape and float(aux["total_loss"]) == 0.0
    # against a direct loop over tokens
    flat = x.reshape(-1, H)
    probs = torch.softmax(blk.router.gate(flat).float(), -1)
    w, idx = probs.topk(k, -1)
    w = w / w.sum(-1, keepdim=True)
    want = torch.zeros_like(flat)
    for t in range(flat.shape[0]):
        for j in range(k):
            e = int(idx[t, j])
            g, u = (flat[t] @ blk.gate_up_proj[e].t()).chunk(2)
            want[t] += w[t, j] * ((F.silu(g) * u) @ blk.down_proj[e].t())
    assert torch.allclose(out.reshape(-1, H), want, atol=1e-4)
    blk.train()
    _, aux = blk(x)
    assert float(aux["aux_loss"]) > 0 and float(aux["z_loss"]) > 0 and float(blk.get_aux_loss()) > 0
    out2, total = K.moe_forward(x, (blk.gate_up_proj, blk.down_proj), blk.router.eval())
    assert torch.allclose(out2, out, atol=1e-5) and float(total) == 0.0

    # the reference's calling convention: cumulative offsets + argsort indices
    rw, sel, offsets, gather, _ = blk.router(x)
    assert offsets[-1] == flat.shape[0] * k and torch.equal(sel.reshape(-1)[gather], sel.reshape(-1)[gather].sort().values)
    W1 = blk.gate_up_proj.detach().clone().requires_grad_(True)
    xin = flat.detach().clone().requires_grad_(True)
    gu = K.MoEGroupedGEMMFunction.apply(xin, W1, k, offsets, gather, None, True, False, False)
    act = F.silu(gu[:, :I]) * gu[:, I:]
    y = K.moe_grouped_gemm_forward(act, blk.down_proj, k, offsets, gather, rw, False, True, True)
    assert torch.allclose(y.view(-1, k, H).sum(1), want, atol=1e-4)
    dgu = torch.randn_like(gu)
    gu.backward(dgu)
    dx = K.moe_grouped_gemm_backward_dx(dgu, W1.detach(), k, offsets, gather, permute_x=True, num_tokens=flat.shape[0])
    dw = K.moe_grouped_gemm_backward_dw(flat, dgu, k, offsets, gather, permute_x=True, num_experts=E)
    assert torch.allclose(dx, xin.grad, atol=1e-4) and torch.allclose(dw, W1.grad, atol=1e-4)
    assert K.get_num_sms() >= 1 and K.get_max_shared_memory() >= 49152 and K.get_l2_cache_size() >= 0
    assert len(K.MoEAutotuneConfig().generate_configs()) == 1
    e = K.ExpertMLPLayer(H, I)
    g_, u_ = e.gate_proj(flat), e.up_proj(flat)
    assert torch.allclose(e(flat), e.down_proj(F.silu(g_) * u_), atol=1e-5)


def test_remaining_kernel_layer_names_against_plain_math():
    import torch.nn as nn
    import torch.nn.functional as F
    torch.manual_seed(3)
    # rotary
    B, S, H, D = 2, 10, 3, 16
    q, k = torch.randn(B, S, H, D), torch.randn(B, S, 1, D)
    rot = K.RotaryEmbedding(D, max_seq_len=8, scaling_type="pi", scaling_factor=2.0)
    q2, k2 = rot.forward_qk(q, k, position_offset=3)
    cos, sin = rot.get_freqs(S + 3)
    assert cos.shape == (S + 3, D // 2)
    c, s_ = cos[3:3 + S][None, :, None, :], sin[3:3 + S][None, :, None, :]
    a, b = q[..., :D // 2], q[..., D // 2:]
    assert torch.allclose(q2, torch.cat((a * c - b * s_, b * c + a * s_), -1), atol=1e-5)
    q3, _ = K.apply_rope_qk(q, k, cos, sin, position_offset=3)
    assert torch.allclose(q3, q2) and torch.allclose(K.RoPEFunction.apply(q, cos, sin, None, 3, False, False), q2)
    assert torch.allclose(rot(q, position_offset=3), q2) and k2.shape == k.shape
    cfg = K.RoPEConfig(dim=D, scaling_type=K.RoPEScalingType.NTK, scaling_factor=4.0)
    assert K.compute_rope_frequencies(cfg, 32)[0].shape == (32, D // 2)
    assert K.get_optimal_block_size(96) == 128 and K.calculate_settings(4096) == (4096, 8)
    assert K.calculate_multi_row_settings(256, 1000)[1] == 8 and K.get_layernorm_info()["max_fused_size"] == 65536
    # norms
    x, r, w = torch.randn(4, 6, 32), torch.randn(4, 6, 32), torch.rand(32) + 0.5
    want = lambda t: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-6) * w   # noqa: E731
    assert torch.allclose(K.rms_layernorm(x, w), want(x), atol=1e-5)
    y, h = K.FusedAddRMSLayerNormFunction.apply(x, r, w, 1e-6, True)
    assert torch.allclose(h, x + r) and torch.allclose(y, want(x + r), atol=1e-5)
    m = K.FusedRMSNorm(32)
    assert torch.allclose(m(x, r), (x + r) * torch.rsqrt((x + r).pow(2).mean(-1, keepdim=True) + 1e-6), atol=1e-5)
    ln = K.LayerNorm(32)
    assert torch.allclose(ln(x), F.layer_norm(x, (32,)), atol=1e-5)
    assert torch.allclose(K.fused_add_layernorm(x, r, ln.weight, ln.bias), F.layer_norm(x + r, (32,)), atol=1e-5)
    assert torch.allclose(K.LayerNormFunction.apply(x, None, None), F.layer_norm(x, (32,)), atol=1e-5)
    # fp8
    spec = K.get_fp8_spec(K.FP8Format.E5M2)
    assert spec.max_val == 57344.0 and spec.exponent_bits == 5
    meta = K.FP8TensorMeta(K.get_fp8_spec("e4m3"), history_len=4)
    for v in (1.0, 8.0, 2.0):
        meta.update_amax(torch.tensor(v))
    sc, inv = meta.compute_scale()
    assert abs(float(sc) - 8.0 / 448.0) < 1e-9 and abs(float(inv) * float(sc) - 1) < 1e-6
    lin = nn.Linear(256, 128)
    net = K.convert_model_to_fp8(nn.Sequential(lin, nn.ReLU(), nn.Linear(128, 128, bias=False)), exclude_layers=["2"])
    xin = torch.randn(5, 256)
    ref = F.linear(xin, lin.weight, lin.bias)
    assert isinstance(net[2], nn.Linear) and not isinstance(net[0], nn.Linear)
    assert (net[0](xin) - ref).abs().max() < 0.05 * ref.abs().max()
    from trainscale_b200.quantization import block_quantize_fp8
    wq, ws = block_quantize_fp8(lin.weight.detach())
    assert (K.fp8_linear_forward(xin, wq, ws, lin.bias) - ref).abs().max() < 0.05 * ref.abs().max()
    assert K.get_fp8_capability()["recommended_block_size"] == 128
    # attention names
    Q, Kt, V = torch.randn(1, 4, 12, 8), torch.randn(1, 2, 12, 8), torch.randn(1, 2, 12, 8)
    i = torch.arange(12)
    o = K.FlashAttentionTritonFunction.apply(Q, Kt, V, True, None, None, 2)
    assert torch.allclose(o, _direct(Q, Kt, V, i[:, None] >= i[None, :], 8 ** -0.5), atol=2e-5)
    assert K.get_attention_backend() in ("tcgen05_flash", "reference") and K.get_flash_attn_version() is None
    # LoRA wrappers
    class L(nn.Module):
        def __init__(s, i, o):
            super().__init__()
            s.weight = nn.Parameter(torch.randn(o, i) * 0.1)
            s.lora_A, s.lora_B, s.scaling = nn.Parameter(torch.randn(4, i) * 0.1), nn.Parameter(torch.randn(o, 4) * 0.1), 0.5
    g_, u_, d_ = L(16, 24), L(16, 24), L(24, 16)
    f = lambda m, t: t @ m.weight.t() + 0.5 * (t @ m.lora_A.t()) @ m.lora_B.t()   # noqa: E731
    xx = torch.randn(7, 16)
    assert torch.allclose(K.FusedLoRAMLP(g_, u_, d_)(xx), f(d_, F.silu(f(g_, xx)) * f(u_, xx)), atol=1e-5)
    assert torch.allclose(K.FusedLoRAQKV(g_, u_, g_)(xx)[1], f(u_, xx), atol=1e-5)
    x24 = torch.randn(3, 24)
    assert torch.allclose(K.apply_lora_o(d_, x24), f(d_, x24), atol=1e-5)
    gate, up, dH = torch.randn(5, 8, requires_grad=True), torch.randn(5, 8, requires_grad=True), torch.randn(5, 8)
    (F.silu(gate) * up).backward(dH)
    hh, d_up, d_gate = K.swiglu_backward(dH, gate.detach(), up.detach())
    assert torch.allclose(d_up, up.grad, atol=1e-6) and torch.allclose(d_gate, gate.grad, atol=1e-6)
    dg2, du2 = K.swiglu_backward_triton(dH, gate.detach(), up.detach())
    assert torch.allclose(dg2, gate.grad, atol=1e-6) and torch.allclose(du2, up.grad, atol=1e-6)
    assert K.dequantize_weight(xx, None) is xx
    # compiler surface: on CPU the wrapper runs eagerly and counts
    @K.compiled()
    def twice(t):
        return t * 2
    assert torch.equal(twice(xx), xx * 2) and twice.stats["eager_calls"] == 1
    with K.compilation_context(disable=True):
        assert torch.equal(K.compile_function(lambda t: t + 1, backend="eager")(xx), xx + 1)
    assert K.get_compiler() is K.get_compiler()
    K.clear_compilation_cache()
    assert K.CUDAGraphConfig().warmup_iterations == 3 and K.InductorConfig().max_autotune and K.DynamicShapeConfig().enabled
