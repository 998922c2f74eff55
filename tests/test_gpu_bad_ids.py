"""Expert ids outside [0,E) through every output mode of the expert pipeline: the permutation drops such
(token,slot) pairs (status bit 0), no kernel indexes with an unwritten position, a dropped slot contributes
nothing to the combined output and its row of the per-slot output is left untouched."""
import pytest
import torch

from oracle import moe_oracle as O
from tests.gpu_util import small_problem, to_dev

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def m():
    import torch_tpu_b200
    torch_tpu_b200.load_ops()
    return torch_tpu_b200


def _problem(T, H, I, E, k):
    p = small_problem(T, H, I, E, k, seed=5)
    ids = p["ids"].clone()
    ids[1, 0] = E                 # one past the end
    ids[T // 2, k - 1] = -1       # negative
    ids[T - 1, 0] = 1 << 30       # far out
    if T > 8:
        ids[5, :] = -7            # a token with no valid slot at all
    p["ids_bad"] = ids
    p["dropped"] = (ids < 0) | (ids >= E)
    return p


@pytest.mark.parametrize("impl", ["simple", "tcgen05"])
@pytest.mark.parametrize("T,H,I,E,k", [(40, 512, 256, 8, 2), (1500, 256, 128, 16, 4)])   # one-CTA and multi-chunk sort
def test_bad_ids_per_slot_and_combined(m, impl, T, H, I, E, k):
    L = m.lib
    p = _problem(T, H, I, E, k)
    d = to_dev(p)
    impl_id = L.IMPL_SIMPLE if impl == "simple" else L.IMPL_TCGEN05
    ids_or, w_or = p["ids_bad"].clone(), p["w"].clone()
    ids_or[p["dropped"]], w_or[p["dropped"]] = 0, 0.0
    # the permutation itself: the tail of sorted_pair is -1, offsets[E] counts the valid pairs only
    sp, off = m.ops.permute(d["ids_bad"], E)
    n_valid = int((~p["dropped"]).sum())
    assert int(off[E].item()) == n_valid and bool((sp[n_valid:] == -1).all()) and bool((sp[:n_valid] >= 0).all())
    # per-slot: dropped rows keep what the caller put there, the others match the oracle
    want = O.experts_w8a8(p["x"], ids_or, p["wg"], p["wu"], p["wd"], p["sg"], p["su"], p["sd"])
    out = torch.full((T, k, H), 7.0, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    m.ops.experts(out, d["x"], d["wg"], d["wu"], d["wd"], d["sg"], d["su"], d["sd"], d["ids_bad"], impl=impl_id,
                  status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == L.STATUS_BAD_EXPERT
    o = out.cpu()
    assert bool((o[p["dropped"]] == 7.0).all())
    met = O.parity_metrics(o[~p["dropped"]], want[~p["dropped"]])
    assert met["max_rel"] <= 2e-2 and met["cosine"] >= 0.9995, met
    # combined (separate kernel) and fused combine: finite, dropped slots contribute nothing
    want_c = O.moe_layer_w8a8(p["x"], ids_or, tuple(p[n] for n in ("wg", "wu", "wd", "sg", "su", "sd")), topk_w=w_or)
    for fused in (False, True):
        y = torch.full((T, H), float("nan"), dtype=torch.bfloat16, device=DEV)
        status.zero_()
        m.ops.experts(y, d["x"], d["wg"], d["wu"], d["wd"], d["sg"], d["su"], d["sd"], d["ids_bad"], d["w"],
                      impl=impl_id, status=status, fused_combine=fused)
        torch.cuda.synchronize()
        assert int(status.item()) == L.STATUS_BAD_EXPERT
        assert bool(torch.isfinite(y.float()).all()), "a dropped slot leaked into the sum"
        met = O.parity_metrics(y.cpu(), want_c)
        assert met["max_rel"] <= 2e-2 and met["cosine"] >= 0.9995, (fused, met)
    if T > 8:
        assert bool((y[5] == 0).all())        # the token without a valid slot gets zeros


def test_op_reports_bad_ids_through_its_status_word(m, monkeypatch):
    T, H, I, E, k = 24, 512, 256, 8, 2
    p = _problem(T, H, I, E, k)
    d = to_dev(p)
    out = torch.zeros(T, k, H, dtype=torch.bfloat16, device=DEV)
    args = (out, d["x"], None, None, d["wg"], d["wu"], d["wd"], d["sg"], d["su"], d["sd"], d["ids_bad"],
            d["w"].to(torch.bfloat16), None, None, None, 128, E, k, False, 1, 1, None, None, None, False)
    word = torch.ops.my_ops.b200_moe_status()
    word.zero_()
    torch.ops.my_ops.fused_moe_fused_experts(*args)      # asynchronous by default: the word carries the report
    torch.cuda.synchronize()
    assert int(word.item()) & 1
    word.zero_()
    monkeypatch.setenv("MOE_CHECK_STATUS", "1")          # debugging switch: synchronise and raise
    with pytest.raises(RuntimeError, match="outside"):
        torch.ops.my_ops.fused_moe_fused_experts(*args)
    assert int(word.item()) == 0                          # cleared after the report
