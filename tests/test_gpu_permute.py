"""Permutation and activation quantisation: integer/byte work, bit-exact against the oracle."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    import torch_tpu_b200
    return torch_tpu_b200.ops


@pytest.mark.parametrize("T,k,E,mode", [
    (1, 1, 1, "rand"), (1, 8, 256, "distinct"), (16, 2, 8, "distinct"), (127, 8, 256, "distinct"),
    (128, 8, 256, "distinct"), (129, 3, 5, "rand"), (1024, 1, 7, "rand"), (1025, 1, 7, "rand"),
    (4096, 2, 8, "distinct"), (8192, 8, 128, "zipf"), (3000, 8, 257, "distinct"), (500, 4, 16, "one_expert"),
    (64, 2, 1000, "distinct")])
def test_permute_bitexact(ops, T, k, E, mode):
    g = torch.Generator().manual_seed(T * 31 + k)
    if mode == "distinct":
        ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])
    elif mode == "rand":
        ids = torch.randint(0, E, (T, k), generator=g)
    elif mode == "one_expert":
        ids = torch.full((T, k), 3)
    else:  # heavy-tailed loads
        p = (torch.arange(1, E + 1).double() ** -1.2)
        ids = torch.multinomial((p / p.sum()).expand(T, E), k, replacement=False, generator=g)
    ids = ids.to(torch.int32)
    want_order, want_offs = O.permutation(ids, E)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    order, offs = ops.permute(ids.to(DEV), E, status=status)
    assert torch.equal(offs.cpu(), want_offs)
    assert torch.equal(order.cpu(), want_order)
    assert int(status.item()) == 0
    # host-side invariants: bijection, counts
    assert torch.equal(torch.sort(order.cpu().long())[0], torch.arange(T * k))
    if mode == "distinct" and E <= 256:
        gather, scatter, cnt = ops.gather_scatter_index(order, offs, T, k, E)
        wg, wsc, wc = O.gather_scatter_index(ids, E)
        assert torch.equal(cnt.cpu(), wc) and torch.equal(gather.cpu(), wg) and torch.equal(scatter.cpu(), wsc)


def test_permute_flags_bad_expert_ids(ops):
    ids = torch.tensor([[0, 9], [1, -1], [2, 1]], dtype=torch.int32)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    order, offs = ops.permute(ids.to(DEV), 4, status=status)
    assert int(status.item()) & 1
    assert offs.cpu().tolist() == [0, 1, 3, 4, 4]
    assert order.cpu()[:4].tolist() == [0, 2, 5, 4]


@pytest.mark.parametrize("T,H,k", [(1, 128, 1), (5, 384, 2), (64, 7168, 8), (1000, 1024, 2)])
def test_quant_rows_bitexact(ops, T, H, k):
    g = torch.Generator().manual_seed(H + T)
    x = (torch.randn(T, H, generator=g) * torch.rand(T, 1, generator=g) * 4).to(torch.bfloat16)
    x[0, :128] = 0  # an all-zero group
    if T > 2:
        x[2, 5] = 300.0  # large outlier
    row_map = torch.randperm(T * k, generator=g).to(torch.int32)
    q, s_t = ops.quant_rows(x.to(DEV), row_map.to(DEV), k)
    wq, ws = O.quant_act_1x128(x[(row_map // k).long()].float())
    assert torch.equal(q.cpu().view(torch.uint8), wq.view(torch.uint8))
    assert torch.equal(s_t.cpu()[:, :T * k].t().contiguous(), ws)
    q2, s2 = ops.quant_rows(x.to(DEV))
    wq2, ws2 = O.quant_act_1x128(x.float())
    assert torch.equal(q2.cpu().view(torch.uint8), wq2.view(torch.uint8))
