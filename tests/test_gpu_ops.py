"""The reference-facing surface: torch.ops.my_ops.* called the way the reference's own tests call them
(python/regression/test_llm/test_moe.py:119-140, test_noaux_tc_topk.py:99-110), and the FusedMoE layer."""
import pytest
import torch

from oracle import moe_oracle as O
from tests.gpu_util import small_problem, to_dev
from tests.helpers import bf16_from_bits, f8_from_bits, load, moe_small_case

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def m():
    import torch_tpu_b200
    torch_tpu_b200.load_ops()
    return torch_tpu_b200


def test_op_noaux_tc_topk_like_reference_test(m):
    z = load("noaux_topk.npz")
    scores = bf16_from_bits(z["ref_scores_bf16"]).repeat(16, 1)
    values = torch.empty(16, 8, dtype=scores.dtype).to(DEV)
    indices = torch.empty(16, 8, dtype=torch.int32).to(DEV)
    torch.ops.my_ops.noaux_tc_topk(values, indices, scores.clone().to(DEV), 8, 4, 8)
    vg, ig = O.noaux_tc_topk(scores, 8, 4, 8)
    assert torch.allclose(vg.float(), values.cpu().float(), rtol=1e-5, atol=1e-6)
    assert torch.equal(ig, indices.cpu().long())
    with pytest.raises(RuntimeError):  # dtype mismatch, as my_ops/NoauxTcTopk.cpp:24-26
        torch.ops.my_ops.noaux_tc_topk(values.float(), indices, scores.to(DEV), 8, 4, 8)
    with pytest.raises(RuntimeError):  # CPU tensors are rejected, there is no CPU path
        torch.ops.my_ops.noaux_tc_topk(values.cpu(), indices.cpu(), scores, 8, 4, 8)


def _call_v1(out, d, E, k):
    return torch.ops.my_ops.fused_moe_fused_experts(
        out, d["x"], None, None, d["wg"], d["wu"], d["wd"], d["sg"], d["su"], d["sd"], d["ids"], d["rw"],
        None, None, None, 128, E, k, True, 8, 4, None, None, None, False)


def test_op_fused_experts_per_slot_and_combined(m):
    T, H, I, E, k = 48, 512, 256, 8, 2
    p = small_problem(T, H, I, E, k, seed=11)
    p["rw"] = p["w"].to(torch.bfloat16)
    d = to_dev(p)
    want = O.experts_w8a8(p["x"], p["ids"], p["wg"], p["wu"], p["wd"], p["sg"], p["su"], p["sd"])
    out = torch.empty(T, k, H, dtype=torch.bfloat16, device=DEV)
    r = _call_v1(out, d, E, k)
    assert r.data_ptr() == out.data_ptr()          # returns the output it was given (my_ops/fusedMoE.cpp:235)
    met = O.parity_metrics(out, want)
    assert met["max_rel"] <= 2e-2 and met["cosine"] >= 0.9995, met
    out2 = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    _call_v1(out2, d, E, k)
    want2 = (want.float() * p["rw"].float()[..., None]).sum(1)
    met = O.parity_metrics(out2, want2)
    assert met["max_rel"] <= 2e-2 and met["cosine"] >= 0.9995, met
    # v2 with the reference's scratch tensors (test_moe.py:289-295)
    sem = torch.empty(E, T, dtype=torch.int32, device=DEV)
    out3 = torch.empty(T, k, H, dtype=torch.bfloat16, device=DEV)
    torch.ops.my_ops.fused_moe_fused_experts_v2(
        out3, d["x"], None, None, d["wg"], d["wu"], d["wd"], d["sg"], d["su"], d["sd"], d["ids"], d["rw"], None,
        sem, sem.clone(), sem.clone(), torch.empty(E, T, k, dtype=torch.int32, device=DEV), 128, E, k, True, 8, 4,
        None, None, None, False)
    assert torch.equal(out3, out)


def test_op_argument_checks(m):
    p = small_problem(4, 256, 128, 4, 2)
    p["rw"] = p["w"].to(torch.bfloat16)
    d = to_dev(p)
    out = torch.empty(4, 2, 256, dtype=torch.bfloat16, device=DEV)
    bad = dict(d)
    bad["ids"] = d["ids"].long()
    with pytest.raises(RuntimeError, match="int32"):   # my_ops/fusedMoE.cpp:143-144
        _call_v1(out, bad, 4, 2)
    with pytest.raises(RuntimeError):
        torch.ops.my_ops.fused_moe_fused_experts(
            out, d["x"], None, None, d["wg"], d["wu"], d["wd"], None, None, None, d["ids"], d["rw"], None, None,
            None, 128, 4, 2, True, 8, 4, None, None, None, False)


def test_op_dense_mlp_w8a16_matches_reference_golden(m):
    z = load("mlp_dense.npz")
    x = bf16_from_bits(z["x"])
    wg, wu, wd = f8_from_bits(z["wg"]), f8_from_bits(z["wu"]), f8_from_bits(z["wd"])
    sg, su, sd = bf16_from_bits(z["sg"]), bf16_from_bits(z["su"]), bf16_from_bits(z["sd"])
    out = torch.empty(x.shape, dtype=torch.bfloat16, device=DEV)
    torch.ops.my_ops.mlp_w8a16_dq_forward(x.to(DEV), wg.to(DEV), wu.to(DEV), wd.t().contiguous().to(DEV),
                                          sg.to(DEV), su.to(DEV), sd.t().contiguous().to(DEV), out, 128)
    met = O.parity_metrics(out.float().flatten(), torch.from_numpy(z["out"].copy()))
    assert met["cos_sim"] >= 0.99 and met["max_rel"] <= 2e-2, met     # test_mlp_w8a16_dq.py:219-220
    out8 = torch.empty_like(out)
    torch.ops.my_ops.mlp_w8a8_quant_forward(x.to(DEV), wg.to(DEV), wu.to(DEV), wd.t().contiguous().to(DEV),
                                            sg.to(DEV), su.to(DEV), sd.t().contiguous().to(DEV), out8, 128)
    met = O.parity_metrics(out8.float().flatten(), torch.from_numpy(z["out"].copy()))
    assert met["cos_sim"] >= 0.99, met


def test_op_fused_moe_grouped_topk(m):
    T, H, E, k = 33, 512, 64, 4
    x, wr, _ = O.make_inputs(T, H, E, seed=2, router_std=0.2)
    ids = torch.empty(T, k, dtype=torch.int32, device=DEV)
    w32 = torch.empty(T, k, dtype=torch.float32, device=DEV)
    w16 = torch.empty(T, k, dtype=torch.bfloat16, device=DEV)
    mm = torch.empty(T, E, dtype=torch.float32, device=DEV)
    sm = torch.empty(T, E, dtype=torch.float32, device=DEV)
    mx = torch.empty(T, dtype=torch.float32, device=DEV)
    xl, wl = x.to(DEV), wr.to(DEV)
    torch.ops.my_ops.fused_moe_grouped_topk(ids, w16, xl, wl, w32, xl.float(), wl.float(), mx, mm, sm)
    O.assert_tie_free(torch.softmax(mm.cpu(), -1), k)
    wid, ww = O.route_softmax_topk(mm.cpu(), k)
    assert torch.equal(ids.cpu(), wid)
    torch.testing.assert_close(w32.cpu(), ww, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("cfgname,T", [("mixtral_like", 80), ("deepseek_like", 80), ("deepseek_like", 24)])
def test_layer_end_to_end(m, cfgname, T):
    from torch_tpu_b200.layer import FusedMoE, MoEConfig
    if cfgname == "mixtral_like":
        cfg = MoEConfig(512, 256, 8, 2)
        bias, shared = None, None
    else:
        cfg = MoEConfig(512, 256, 64, 6, "sigmoid", 8, 4, True, 2.5, shared_intermediate=256)
        bias = torch.randn(64, generator=torch.Generator().manual_seed(1)) * 0.01
        shared = O.make_expert_weights(1, 512, 256, seed=77)
    # T = 24 with a shared expert takes the decode-size route: shared expert on the side stream, K split over CTAs
    p = small_problem(T, cfg.hidden, cfg.intermediate, cfg.num_experts, cfg.top_k, seed=21)
    x, wr, _ = O.make_inputs(T, cfg.hidden, cfg.num_experts, seed=21, router_std=0.2)
    layer = FusedMoE(cfg, wr.to(DEV), *(p[n].to(DEV) for n in ("wg", "wu", "wd", "sg", "su", "sd")),
                     bias=bias.to(DEV) if bias is not None else None,
                     shared=tuple(t.to(DEV) for t in shared) if shared else None, max_tokens=128)
    y = layer(x.to(DEV))
    ids, w = layer.ids[:T].cpu(), layer.topk_w[:T].cpu()
    lg = layer.logits[:T].cpu()
    if cfgname == "mixtral_like":
        wid, ww = O.route_softmax_topk(lg, cfg.top_k)
    else:
        wid, ww = O.route_sigmoid_grouped(lg, bias, 8, 4, cfg.top_k, 2.5)
    assert torch.equal(ids, wid)
    want = O.moe_layer_w8a8(x, wid, tuple(p[n] for n in ("wg", "wu", "wd", "sg", "su", "sd")),
                            shared=tuple(t[0] for t in shared) if shared else None, topk_w=w)
    met = O.parity_metrics(y, want)
    assert met["max_rel"] <= 2e-2 and met["cosine"] >= 0.9995, met
    assert int(layer.status.item()) == 0
    # CUDA-graph replay gives the same bits
    yg = layer.forward_graph(x.to(DEV))
    torch.cuda.synchronize()
    same = torch.equal if T > 64 else (lambda a, b: bool(((a.float() - b.float()).abs() <= 1e-2 * b.float().abs() + 1e-3).all()))
    assert same(yg, y)   # split-K partial sums are added in arrival order, so only the unsplit route is bit-stable
    # host-buffer entry point
    xh, oh = x.pin_memory(), torch.empty(T, cfg.hidden, dtype=torch.bfloat16).pin_memory()
    for _ in range(3):   # pipelined: two buffers each way
        layer.forward_host(xh, oh)
    layer.host_join()
    torch.cuda.synchronize()
    assert same(oh, y.cpu())


@pytest.mark.parametrize("M,K,N", [(32, 7168, 1536), (32, 7168, 576), (32, 2048, 7168), (64, 4096, 2048),
                                   (300, 512, 320)])
def test_mm_w8a16_dq_forward(m, M, K, N):
    """Dense block-scaled linear layer through the reference's op name, on the reference's own shapes and input
    distributions (python/regression/test_llm/test_mm_w8a16_dq.py:101-140: randn activations, randn weights cast to
    e4m3, randn bf16 scales).  Expected value: the reference's CPU function (dequantise the weight block-wise,
    F.linear) on the activations as the kernel sees them (quantised 1x128, tolerance of the FP8 path), and the
    reference's own acceptance metric against the unquantised activations."""
    g = torch.Generator().manual_seed(M + K + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g).to(torch.float8_e4m3fn)
    s = torch.randn((N + 127) // 128, (K + 127) // 128, generator=g).to(torch.bfloat16)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    r = torch.ops.my_ops.mm_w8a16_dq_forward(x.to(DEV), w.to(DEV), s.to(DEV), out, 128)
    assert r.data_ptr() == out.data_ptr()
    wd = (w.float().view(-1) .view(N, K))
    sb = s.float().repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
    wdq = wd * sb                                           # fp32 dequantised weight
    xq, xs = O.quant_act_1x128(x)
    want_q = O.dequant_act(xq, xs).double() @ wdq.double().T
    met = O.parity_metrics(out.cpu(), want_q)
    assert met["max_rel"] <= 2e-2 and met["cosine"] >= 0.9995, met
    want_ref = x.float().double() @ wdq.double().T          # the reference's arithmetic: bf16 activations
    assert O.cos_sim(out.cpu().float().numpy(), want_ref.numpy()) > 0.99


@pytest.mark.parametrize("M,K,N", [(500, 4096, 8192), (64, 512, 320), (1, 128, 64)])
def test_scaled_mm_fp8(m, M, K, N):
    """FP8 x FP8 product with one scale per operand, on the reference's own shape and input distribution
    (python/test/_scaled_mm.py:39-44,80: uniform [-1,1] cast to e4m3, scales 1) plus non-trivial scales; expected value
    = the fp32 product of the e4m3 values (every partial product is exact, so only fp32 summation order differs)."""
    g = torch.Generator().manual_seed(1000)
    x = (torch.rand(M, K, generator=g) * 2 - 1).to(torch.float8_e4m3fn)
    y = (torch.rand(K, N, generator=g) * 2 - 1).to(torch.float8_e4m3fn)
    want = x.float().double() @ y.float().double()
    for sa, sb, dt in ((1.0, 1.0, torch.float32), (0.5, 3.0, torch.float32), (0.25, 2.0, torch.bfloat16)):
        out = torch.ops.my_ops._scaled_mm(x.to(DEV), y.t().contiguous().to(DEV), torch.tensor(sa), torch.tensor(sb),
                                          None, None, dt, False)
        assert out.dtype == dt and tuple(out.shape) == (M, N)
        met = O.parity_metrics(out.cpu(), want * sa * sb)
        tol = 1e-5 if dt == torch.float32 else 4e-3
        assert met["max_rel"] <= tol and met["cosine"] >= 0.99999, (sa, sb, dt, met)
        # the reference's acceptance test: row-wise cosine >= 0.99 (python/test/_scaled_mm.py:62-65)
        cs = torch.nn.functional.cosine_similarity(out.cpu().double(), want * sa * sb, dim=1)
        assert float(cs.min()) >= 0.99


def test_profile_toggles_like_the_reference(m):
    """enable_profile / disable_profile (torch_tpu/csrc/ops/my_ops/myOps.cpp:67-68; called as
    torch.ops.my_ops.enable_profile(4096, mode) in python/tgi_test/tgi_modules.py:192): while enabled every op call
    is timed with CUDA events on the current stream; disable_profile() prints and keeps calls / total / average per op.
    Calls made while disabled are not counted; max_record_num bounds the timed calls."""
    z = load("noaux_topk.npz")
    scores = bf16_from_bits(z["ref_scores_bf16"]).repeat(16, 1).to(DEV)
    values = torch.empty(16, 8, dtype=scores.dtype, device=DEV)
    indices = torch.empty(16, 8, dtype=torch.int32, device=DEV)
    call = lambda: torch.ops.my_ops.noaux_tc_topk(values, indices, scores, 8, 4, 8)
    call()                                           # not counted: profiling is off
    torch.ops.my_ops.enable_profile(4096, 1)
    for _ in range(5):
        call()
    torch.ops.my_ops.disable_profile()
    call()                                           # not counted either
    rows = [r.strip().split(", ") for r in torch.ops.my_ops.b200_profile_summary().splitlines()[1:]]
    assert len(rows) == 1 and rows[0][0] == "noaux_tc_topk" and int(rows[0][1]) == 5
    assert 0.0 < float(rows[0][2]) < 1000.0 and float(rows[0][3]) > 0.0
    torch.ops.my_ops.enable_profile(2, None)         # only the first two calls are timed
    for _ in range(4):
        call()
    torch.ops.my_ops.disable_profile()
    rows = [r.strip().split(", ") for r in torch.ops.my_ops.b200_profile_summary().splitlines()[1:]]
    assert int(rows[0][1]) == 2
