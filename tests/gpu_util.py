"""Helpers of the GPU parity tests: move oracle-generated inputs to the device, run, compare."""
import torch

from oracle import moe_oracle as O


def small_problem(T, H, I, E, k, seed=0, distinct=True, scale_dtype=torch.float32):
    """Seeded synthetic problem generated ON THE CPU (identical bits for oracle and device)."""
    wg, wu, wd, sg, su, sd = O.make_expert_weights(E, H, I, seed)
    x, wr, logits = O.make_inputs(T, H, E, seed)
    g = torch.Generator().manual_seed(seed + 99)
    if distinct:
        ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32) if T else \
            torch.zeros(0, k, dtype=torch.int32)
    else:
        ids = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32)
    w = torch.rand(T, k, generator=g) + 0.1
    w = w / w.sum(-1, keepdim=True)
    if scale_dtype != torch.float32:
        sg, su, sd = sg.to(scale_dtype), su.to(scale_dtype), sd.to(scale_dtype)
    return dict(x=x, wr=wr, logits=logits, ids=ids, w=w, wg=wg, wu=wu, wd=wd, sg=sg, su=su, sd=sd)


def to_dev(p, dev="cuda:0"):
    return {k: (v.to(dev).contiguous() if isinstance(v, torch.Tensor) else v) for k, v in p.items()}
