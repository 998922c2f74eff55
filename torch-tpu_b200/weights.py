"""Weight preparation for the fused-MoE op: FP8 block quantisation and the checkpoint-layout -> op-layout
conversion.  This is set-up code (runs once per model load, plain torch ops on whatever device the tensors are
on); the per-token hot path never comes here.

Op layout (what the reference's device op consumes, python/regression/test_llm/test_moe.py:282-288 and
torch_tpu/csrc/ops/native_ops/CopyFrom.cpp:598-599):
  gate, up  : [E, I, H] float8_e4m3fn
  down      : [E, I, H] float8_e4m3fn  = W_down^T, CONTIGUOUS (a strided transpose view is not accepted)
  scales    : [E, ceil(I/128), ceil(H/128)] float32 (bfloat16 also accepted by the op)
"""
import torch

BLOCK = 128
FP8_MAX = 448.0


def quantize_blockwise(w: torch.Tensor, block: int = BLOCK):
    """[..., R, C] float -> (e4m3 [..., R, C], fp32 scale [..., ceil(R/b), ceil(C/b)]), scale = block amax / 448."""
    *lead, R, C = w.shape
    nr, nc = (R + block - 1) // block, (C + block - 1) // block
    wp = torch.zeros(*lead, nr * block, nc * block, dtype=torch.float32, device=w.device)
    wp[..., :R, :C] = w.to(torch.float32)
    blk = wp.view(*lead, nr, block, nc, block)
    amax = blk.abs().amax(dim=(-3, -1)).clamp_min(1e-12)
    s = amax / FP8_MAX
    q = (blk / s[..., :, None, :, None]).clamp(-FP8_MAX, FP8_MAX).view(*lead, nr * block, nc * block)[..., :R, :C]
    return q.to(torch.float8_e4m3fn).contiguous(), s.contiguous()


def dequantize_blockwise(q: torch.Tensor, s: torch.Tensor, block: int = BLOCK, dtype=torch.float32):
    *lead, R, C = q.shape
    sf = s.to(torch.float32).repeat_interleave(block, -2)[..., :R, :].repeat_interleave(block, -1)[..., :C]
    return (q.to(torch.float32) * sf).to(dtype)


def experts_from_checkpoint(gate_proj, up_proj, down_proj, gate_scale=None, up_scale=None, down_scale=None):
    """Per-expert lists (or stacked tensors) in the usual checkpoint layout - gate_proj/up_proj [I,H], down_proj [H,I],
    block scales (``weight_scale_inv``) [ceil(rows/128), ceil(cols/128)] - to the op layout.  bf16/fp32 weights
    without scales are block-quantised here; FP8 weights keep their bytes and scales and only the down projection
    (and its scale grid) is transposed and made contiguous."""
    def stack(v):
        return torch.stack(list(v)) if not isinstance(v, torch.Tensor) else v

    g, u, d = stack(gate_proj), stack(up_proj), stack(down_proj)
    if g.dtype == torch.float8_e4m3fn:
        if gate_scale is None or up_scale is None or down_scale is None:
            raise ValueError("FP8 checkpoint weights need their block scales")
        sg, su, sd = stack(gate_scale).float(), stack(up_scale).float(), stack(down_scale).float()
        return (g.contiguous(), u.contiguous(), d.transpose(-1, -2).contiguous(), sg.contiguous(), su.contiguous(),
                sd.transpose(-1, -2).contiguous())
    gq, sg = quantize_blockwise(g)
    uq, su = quantize_blockwise(u)
    dq, sd = quantize_blockwise(d.transpose(-1, -2))
    return gq, uq, dq, sg, su, sd


def random_experts(E, H, I, device, seed=0, std=0.02, chunk=8):
    """Seeded N(0,std) expert weights quantised on ``device`` (benchmark inputs).  Generated ``chunk`` experts at a
    time so that the fp32 staging stays small next to the FP8 result."""
    g = torch.Generator(device=device).manual_seed(seed)
    nI, nH = (I + BLOCK - 1) // BLOCK, (H + BLOCK - 1) // BLOCK
    out = [torch.empty(E, I, H, dtype=torch.float8_e4m3fn, device=device) for _ in range(3)]
    sc = [torch.empty(E, nI, nH, dtype=torch.float32, device=device) for _ in range(3)]
    for e0 in range(0, E, chunk):
        n = min(chunk, E - e0)
        for m in range(3):
            w = torch.randn(n, I, H, generator=g, device=device, dtype=torch.float32) * std
            q, s = quantize_blockwise(w)
            out[m][e0:e0 + n], sc[m][e0:e0 + n] = q, s
            del w, q, s
    return (*out, *sc)
