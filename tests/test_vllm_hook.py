"""The linear-method hook (counterpart of the reference's vLLM plugin patch): host logic on the CPU with
a stand-in method class and module factory, and the real modules on the GPU."""
import pytest
import torch

from quadbit_b200 import vllm_hook


class FakeMethod:
    """The two methods a serving engine's linear method has."""

    def __init__(self):
        self.pw_calls = 0

    def process_weights_after_loading(self, layer):
        self.pw_calls += 1

    def apply(self, layer, x, bias=None):
        y = torch.nn.functional.linear(x, layer.weight)
        return y + bias if bias is not None else y


class FakeLayer:
    def __init__(self, out_f, in_f, device="cpu"):
        self.weight = torch.nn.Parameter(torch.randn(out_f, in_f, device=device) * 0.02, requires_grad=False)


class Recorder:
    def __init__(self, w):
        self.w = w.float()

    def forward(self, x):
        return torch.nn.functional.linear(x.float(), self.w).to(torch.bfloat16)


def test_hook_patches_and_restores_on_cpu():
    for k in vllm_hook.STATS:
        vllm_hook.STATS[k] = 0
    restore = vllm_hook.install(FakeMethod, mode="sparse", factory=Recorder)
    try:
        m = FakeMethod()
        good, odd = FakeLayer(256, 128), FakeLayer(100, 128)
        m.process_weights_after_loading(good)
        m.process_weights_after_loading(odd)
        assert m.pw_calls == 2                                   # the engine's own step still runs
        assert isinstance(good._qb_linear, Recorder) and not hasattr(odd, "_qb_linear")
        assert vllm_hook.STATS["sparse_layers"] == 1 and vllm_hook.STATS["native_layers"] == 1
        x = torch.randn(3, 5, 128)
        b = torch.randn(256)
        y = m.apply(good, x, b)
        assert y.shape == (3, 5, 256) and y.dtype == x.dtype
        assert torch.allclose(y, torch.nn.functional.linear(x, good.weight) + b, atol=2e-2)
        y2 = m.apply(odd, x[..., :128])                          # untouched layer: engine path
        assert torch.allclose(y2, torch.nn.functional.linear(x, odd.weight))
        assert vllm_hook.STATS["calls"] == 1
    finally:
        restore()
    assert FakeMethod.apply.__name__ == "apply" and "patched" not in FakeMethod.process_weights_after_loading.__name__


def test_hook_select_and_mode_validation():
    with pytest.raises(ValueError):
        vllm_hook.install(FakeMethod, mode="fp8")
    restore = vllm_hook.install(FakeMethod, mode="dense", factory=Recorder, select=lambda layer: False)
    try:
        layer = FakeLayer(128, 128)
        FakeMethod().process_weights_after_loading(layer)
        assert not hasattr(layer, "_qb_linear")
    finally:
        restore()


def test_install_vllm_needs_a_resolvable_class():
    with pytest.raises((ImportError, AttributeError)):
        vllm_hook.install_vllm(method="no_such_engine.layers.LinearMethod")


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["sparse", "dense"])
def test_hook_runs_the_gpu_modules(mode):
    import quadbit_b200 as qb
    torch.manual_seed(5)
    restore = vllm_hook.install(FakeMethod, mode=mode)
    try:
        m = FakeMethod()
        layer = FakeLayer(512, 1024, device="cuda")
        m.process_weights_after_loading(layer)
        x = torch.randn(2, 70, 1024, device="cuda", dtype=torch.bfloat16)
        bias = torch.randn(512, device="cuda", dtype=torch.bfloat16)
        y = m.apply(layer, x, bias)
        ref_mod = (qb.QuadbitLinear if mode == "sparse" else qb.DenseNVLinear)(layer.weight.data, keep_ref_layout=False)
        assert torch.equal(y, ref_mod.forward(x).to(x.dtype) + bias)
        assert y.shape == (2, 70, 512)
    finally:
        restore()


class FakeMoEMethod:
    """The two methods of a serving engine's fused-MoE method."""

    def process_weights_after_loading(self, layer):
        layer.seen = True

    def apply(self, layer, x, topk_weights, topk_ids, shared_experts=None, shared_experts_input=None):
        raise AssertionError("the engine's own MoE path must not run for a packed layer")


@pytest.mark.gpu
def test_moe_method_hook_from_mxfp4_expert_tensors():
    """install_moe on a stand-in method class: gpt-oss-style MXFP4 expert tensors (interleaved gate / up rows, e8m0 per 32)
    are dequantised, pruned and packed once; apply() equals a SparseMoE built by hand from the dequantised weights."""
    import quadbit_b200 as qb
    from oracle import fakequant as fq
    torch.manual_seed(9)
    E, H, I, T, topk = 4, 256, 128, 40, 2

    class Layer:
        pass

    layer = Layer()
    layer.w13_weight = torch.randint(0, 256, (E, 2 * I, H // 2), dtype=torch.int32).to(torch.uint8).cuda()
    layer.w13_weight_scale = torch.randint(118, 124, (E, 2 * I, H // 32), dtype=torch.int32).to(torch.uint8).cuda()
    layer.w2_weight = torch.randint(0, 256, (E, H, I // 2), dtype=torch.int32).to(torch.uint8).cuda()
    layer.w2_weight_scale = torch.randint(118, 124, (E, H, I // 32), dtype=torch.int32).to(torch.uint8).cuda()
    restore = vllm_hook.install_moe(FakeMoEMethod, fmt="mxfp4", act="gptoss")
    try:
        m = FakeMoEMethod()
        m.process_weights_after_loading(layer)
        assert layer.seen and isinstance(layer._qb_moe, qb.SparseMoE)
        x = torch.randn(T, H).cuda().bfloat16()
        idx, w = fq.route_topk(torch.randn(T, E), topk)
        y = m.apply(layer, x, w.cuda(), idx.cuda())
    finally:
        restore()
    gus, dns = [], []
    for e in range(E):
        w13 = fq.mxfp4_dequant(layer.w13_weight[e].cpu(), layer.w13_weight_scale[e].cpu())
        gus.append(torch.cat([w13[0::2], w13[1::2]], 0).cuda())
        dns.append(fq.mxfp4_dequant(layer.w2_weight[e].cpu(), layer.w2_weight_scale[e].cpu()).cuda())
    ref = qb.SparseMoE(gus, dns, topk, act="gptoss").forward(x, idx.cuda(), w.cuda())
    assert y.shape == (T, H) and torch.equal(y, ref)
    assert FakeMoEMethod.apply is not None and vllm_hook.STATS["moe_calls"] >= 1


@pytest.mark.gpu
def test_moe_method_hook_applies_expert_biases():
    """gpt-oss layers carry w13_bias / w2_bias: the hook hands them to the epilogues of the grouped GEMMs
    (gate/up + bias before the clamped SwiGLU, (down + bias) * routing weight). Checked against a per-expert loop of the
    CPU oracle with the same bf16 roundings."""
    from oracle import fakequant as fq
    torch.manual_seed(10)
    E, H, I, T, topk = 4, 256, 128, 48, 2

    class Layer:
        pass

    layer = Layer()
    w13 = (torch.randn(E, 2 * I, H) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I) * 0.05).to(torch.bfloat16)
    b13 = (torch.randn(E, 2 * I) * 0.3).to(torch.bfloat16)
    b2 = (torch.randn(E, H) * 0.3).to(torch.bfloat16)
    layer.w13_weight, layer.w2_weight, layer.w13_bias, layer.w2_bias = w13.cuda(), w2.cuda(), b13.cuda(), b2.cuda()
    restore = vllm_hook.install_moe(FakeMoEMethod, fmt="bf16", act="gptoss")
    try:
        m = FakeMoEMethod()
        m.process_weights_after_loading(layer)
        x = torch.randn(T, H).to(torch.bfloat16)
        idx, w = fq.route_topk(torch.randn(T, E), topk)
        y = m.apply(layer, x.cuda(), w.cuda(), idx.cuda()).float().cpu()
        with pytest.raises(NotImplementedError):
            m.apply(layer, x.cuda(), w.cuda(), idx.cuda(), expert_map=torch.arange(E))
    finally:
        restore()
    ref = torch.zeros(T, H)
    for e in range(E):
        sel = idx == e
        toks = torch.nonzero(sel.any(1)).squeeze(1)
        if toks.numel() == 0:
            continue
        gu = (fq.linear_sparse(x[toks].float(), w13[e].float()) + b13[e].float()).to(torch.bfloat16).float()
        g, u = gu[:, :I].clamp(max=7.0), gu[:, I:].clamp(-7.0, 7.0)
        h = (g * torch.sigmoid(1.702 * g)) * (u + 1.0)
        d = F_linear_2lvl(fq, h, w2[e].float())
        wt = (w * sel)[toks].sum(1, keepdim=True)
        ref[toks] += ((d + b2[e].float()) * wt).to(torch.bfloat16).float()
    assert ((y - ref).norm() / ref.norm()).item() < 0.03
    bias_effect = (b2.float().abs().mean() / ref.abs().mean()).item()
    assert bias_effect > 0.05           # the biases are large enough that leaving them out would fail the bound above


def F_linear_2lvl(fq, h, w):
    """Down projection of the layer: h is quantised in fp32 (no bf16 rounding) by the SwiGLU quantiser."""
    return torch.nn.functional.linear(fq.act_dequant_2lvl(h, 32, round_bf16=False), fq.sparse_fp4_dequant_2lvl(w))
