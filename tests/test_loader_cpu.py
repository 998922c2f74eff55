"""The weight-layout loader (torch-tpu_b200/weights.py): checkpoint-layout tensors -> the layout the fused-MoE op
consumes.  What the reference's test does by hand before it calls the device op
(python/regression/test_llm/test_moe.py:282-288: the down projection and its scale grid transposed, the transposes
made contiguous by the copy to the device, torch_tpu/csrc/ops/native_ops/CopyFrom.cpp:598-599) must come out of
``experts_from_checkpoint`` byte for byte, and feeding the result to the oracle must reproduce the reference's own
stored outputs."""
import numpy as np
import torch

from oracle import moe_oracle as O
from tests.helpers import bf16_from_bits, f8_from_bits, load, moe_small_case


def _weights_module():
    import torch_tpu_b200
    return torch_tpu_b200.weights


def test_fp8_checkpoint_layout_matches_the_reference_hand_built_layout():
    W = _weights_module()
    for name in ("a", "b"):
        z = load("moe_small.npz")
        w0, w1, w2 = (f8_from_bits(z[f"{name}_w{i}"]) for i in range(3))       # gate/up [E,I,H], down [E,H,I]
        s0, s1, s2 = (bf16_from_bits(z[f"{name}_s{i}"]) for i in range(3))     # [E,nI,nH] x2, [E,nH,nI]
        E = w0.shape[0]
        # per-expert lists, as a checkpoint reader hands them over
        got = W.experts_from_checkpoint([w0[e] for e in range(E)], [w1[e] for e in range(E)],
                                        [w2[e] for e in range(E)], [s0[e] for e in range(E)],
                                        [s1[e] for e in range(E)], [s2[e] for e in range(E)])
        c = moe_small_case(name)                                              # the hand-built device layout
        for g, key in zip(got[:3], ("wg", "wu", "wd")):
            assert g.is_contiguous() and g.dtype == torch.float8_e4m3fn
            assert torch.equal(g.view(torch.uint8), c[key].view(torch.uint8)), key
        for g, key in zip(got[3:], ("sg", "su", "sd")):
            assert g.is_contiguous() and g.dtype == torch.float32
            assert torch.equal(g, c[key].float()), key                        # bf16 -> fp32 is exact
        # the op layout feeds the oracle: the reference's stored outputs come back bit for bit
        out = O.experts_w8a16(c["x"], c["ids"], got[0], got[1], got[2], *(t.to(torch.bfloat16) for t in got[3:]),
                              per_token=True)
        assert torch.equal(out, c["out"])


def test_unquantised_checkpoint_is_block_quantised_with_amax_over_448():
    W = _weights_module()
    g = torch.Generator().manual_seed(11)
    E, H, I = 3, 384, 200                                    # I not a multiple of 128: ragged last block row
    gate = torch.randn(E, I, H, generator=g) * 0.02
    up = torch.randn(E, I, H, generator=g) * 0.02
    down = torch.randn(E, H, I, generator=g) * 0.02          # checkpoint layout of the down projection
    wg, wu, wd, sg, su, sd = W.experts_from_checkpoint(gate.to(torch.bfloat16), up.to(torch.bfloat16),
                                                       down.to(torch.bfloat16))
    nI, nH = (I + 127) // 128, H // 128
    assert wg.shape == (E, I, H) and wd.shape == (E, I, H) and wd.is_contiguous()
    assert sg.shape == (E, nI, nH) and sd.shape == (E, nI, nH) and sd.dtype == torch.float32
    # scale = block amax / 448 of the bf16 weights; the same rule as the oracle's quantiser
    for e in range(E):
        q, s = O.quant_weight_128x128(gate[e].to(torch.bfloat16).float())
        assert torch.equal(q.view(torch.uint8), wg[e].view(torch.uint8)) and torch.equal(s, sg[e])
        q, s = O.quant_weight_128x128(down[e].to(torch.bfloat16).float().t().contiguous())
        assert torch.equal(q.view(torch.uint8), wd[e].view(torch.uint8)) and torch.equal(s, sd[e])
    # dequantising gives the weights back to within half an e4m3 step of each block's range
    back = W.dequantize_blockwise(wd, sd)
    want = down.to(torch.bfloat16).float().transpose(1, 2)
    step = sd.repeat_interleave(128, 1)[:, :I].repeat_interleave(128, 2) * 32.0   # largest e4m3 spacing: 32 at 256..448
    assert bool(((back - want).abs() <= 0.5 * step * (1 + 1e-5) + 1e-12).all())


def test_fp8_checkpoint_without_scales_is_rejected():
    W = _weights_module()
    w = torch.zeros(1, 128, 128).to(torch.float8_e4m3fn)
    try:
        W.experts_from_checkpoint(w, w, w)
    except ValueError as exc:
        assert "scales" in str(exc)
    else:
        raise AssertionError("expected a ValueError")
