"""Generates the golden fixtures in this directory by running the reference's own torch oracle.

Run once where a checkout of the reference project is available (pass its root as argv[1] or in the environment variable
``AMD_KERNELS_REFERENCE``):  ``python tests/golden/make_golden.py REFERENCE_ROOT``.  Machines that run the tests need no
reference checkout; tests read only the ``.npz`` files written here. ``reference.py`` is loaded by file path because the package's
``__init__`` imports the AMD JIT toolchain.

Fixtures (inputs are stored or re-derivable from the stated seed; outputs come from the reference functions named):
  quant.npz    bf16 rows with one binade per 32-block, zero blocks, many E2M1 midpoints (recipe of the reference's
               tests/moe/.../test_quant.py:25-31)            -> mxfp4_quant_ref, dequant_mxfp4
  routing.npz  fp32 logits / split-K partials incl. exact ties -> splitk_logits_reference, biased_topk_reference, decided
  swiglu.npz   fp32 gate / up                                  -> swiglu_oai
  reduce.npz   bf16 slots incl. signed zeros and subnormals    -> reduce_slots_bf16_ref
  moe_small.npz  E=8, H=256, I=64, T=32 MXFP4 layer            -> w4a4_moe_ref
  shared.npz   bf16 rows -> shared_mxfp8_quant_ref; seeded MXFP8 weights -> shared_mxfp8_ref; torch's E4M3 cast
  sidecar.npz  bf16 rows -> both quantisers -> mxfp4_sidecar_pack_ref (mask) and mxfp4_sidecar_unpack_ref (== the FP4 codes)
  tail.npz     bf16 slots / shared / residual / norm weight -> slots4_local_reference, add_rmsnorm_reference,
               mxfp8_scale_reference, mxfp8_codes of amd_kernels/norm/gemma_add_rmsnorm_h6144/reference.py (the contract of
               the fused MoE tail, amd_kernels/collectives/pull_collectives_ranks4/reference.py:74-91 for the slot sum)
  moe_config0.npz  the benchmark's configuration 0 (T=16, E=128, H=6144, I=768, seed 0; inputs re-derived from the seed
               by oracle.moe_oracle.make_weights / make_inputs, their CRC32 stored) -> w4a4_moe_ref on softmax top-4
               routing, and on the reference's sigmoid+bias routing
"""
import importlib.util
import os
import sys
import zlib

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle import moe_oracle as orc  # noqa: E402


def load_reference(root):
    path = os.path.join(root, "amd_kernels/moe/mxfp4_h6144_i768_e128_top4/reference.py")
    spec = importlib.util.spec_from_file_location("reference_moe", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load_norm_reference(root):
    path = os.path.join(root, "amd_kernels/norm/gemma_add_rmsnorm_h6144/reference.py")
    spec = importlib.util.spec_from_file_location("reference_norm", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def bits(t):
    return t.view(torch.int16).numpy().view(np.uint16).copy()


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("AMD_KERNELS_REFERENCE")
    if not root:
        raise SystemExit("usage: make_golden.py REFERENCE_ROOT (or set AMD_KERNELS_REFERENCE)")
    ref = load_reference(root)
    torch.set_num_threads(os.cpu_count())

    # ---- quant
    g = torch.Generator().manual_seed(8)
    m, hidden = 8, 6144
    x = torch.randn((m, hidden // 32, 32), generator=g)
    x *= torch.exp2(torch.randint(-20, 21, (m, hidden // 32, 1), generator=g).float())
    x[torch.rand((m, hidden // 32), generator=g) < 0.02] = 0.0
    x = x.view(m, hidden).bfloat16()
    x[0, :32] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 7.0, -0.0, -0.25, -0.75, -6.5, 4.0, 3.0, 0.5] * 2)
    q, s = ref.mxfp4_quant_ref(x)
    f32 = torch.randn((4, 768), generator=g) * 3.0  # the GEMM1 epilogue quantizes fp32, not bf16
    q32, s32 = ref.mxfp4_quant_ref(f32)
    np.savez_compressed(os.path.join(HERE, "quant.npz"), x_bits=bits(x), codes=q.numpy(), scales=s.numpy(),
                        deq=ref.dequant_mxfp4(q, s).numpy(), f32=f32.numpy(), codes32=q32.numpy(), scales32=s32.numpy())

    # ---- routing
    g = torch.Generator().manual_seed(5)
    n, splits = 64, 16
    parts = torch.randn((splits, n, 128), generator=g)
    parts[:, 0] = 0.25
    parts[:, 1, 3:40] = 0.5
    parts[:, 2] = parts[:, 2, :8].repeat(1, 16)
    parts[:, n - 1, ::5] = 1.0
    parts = parts.permute(1, 0, 2).contiguous()
    logits = ref.splitk_logits_reference(parts)
    bias = torch.randn((128,), generator=g) * 0.1
    bias[::7] = 0.0
    w, ids, vals = ref.biased_topk_reference(logits, bias, 4, 2.0)
    np.savez_compressed(os.path.join(HERE, "routing.npz"), partials=parts.numpy(), logits=logits.numpy(),
                        bias=bias.numpy(), weights=w.numpy(), ids=ids.numpy(), vals=vals.numpy(),
                        decided=ref.decided(vals).numpy())

    # ---- swiglu
    g = torch.Generator().manual_seed(6)
    gate, up = torch.randn((64, 96), generator=g) * 5, torch.randn((64, 96), generator=g) * 5
    np.savez_compressed(os.path.join(HERE, "swiglu.npz"), gate=gate.numpy(), up=up.numpy(),
                        out=ref.swiglu_oai(gate, up).numpy())

    # ---- reduce
    g = torch.Generator().manual_seed(7)
    slots = (torch.randn((8, 4, 6144), generator=g) * torch.exp2(torch.randint(-130, 20, (8, 4, 1), generator=g).float())
             ).bfloat16()
    slots[0, :, :16] = 0.0
    slots[0, 1, :8] = -0.0
    slots[1, :, :4] = -0.0
    np.savez_compressed(os.path.join(HERE, "reduce.npz"), slots=bits(slots), out=bits(ref.reduce_slots_bf16_ref(slots)))

    # ---- small MoE
    (w13, s13, w2, s2), gen = orc.make_weights(seed=3, experts=8, hidden=256, inter=64)
    xb, lg = orc.make_inputs(gen, 32, hidden=256, experts=8)
    xq, xs = ref.mxfp4_quant_ref(torch.from_numpy(orc.bf16_to_f32(xb)))
    wts, tid, _ = orc.route_softmax(lg)
    out = ref.w4a4_moe_ref((xq, xs), *(torch.from_numpy(a) for a in (w13, s13, w2, s2)),
                           torch.from_numpy(wts.astype(np.float32)), torch.from_numpy(tid))
    np.savez_compressed(os.path.join(HERE, "moe_small.npz"), w13=w13, s13=s13, w2=w2, s2=s2, x_bits=xb, logits=lg,
                        weights=wts.astype(np.float32), ids=tid.astype(np.int32), out=out.numpy())

    # ---- configuration 0 at full shape
    (w13, s13, w2, s2), gen = orc.make_weights(seed=0)
    xb, lg = orc.make_inputs(gen, 16)
    crc = np.array([zlib.crc32(a.tobytes()) for a in (w13, s13, w2, s2, xb, lg)], dtype=np.uint32)
    xq, xs = ref.mxfp4_quant_ref(torch.from_numpy(orc.bf16_to_f32(xb)))
    tw = [torch.from_numpy(a) for a in (w13, s13, w2, s2)]
    wts, tid, _ = orc.route_softmax(lg)
    out_soft = ref.w4a4_moe_ref((xq, xs), *tw, torch.from_numpy(wts.astype(np.float32)), torch.from_numpy(tid))
    bias = torch.zeros(128)
    wsig, isig, vsig = ref.biased_topk_reference(torch.from_numpy(lg), bias, 4, 2.0)
    out_sig = ref.w4a4_moe_ref((xq, xs), *tw, wsig.float(), isig)
    np.savez_compressed(os.path.join(HERE, "moe_config0.npz"), crc=crc, xq=xq.numpy(), xs=xs.numpy(),
                        weights_softmax=wts.astype(np.float32), ids_softmax=tid.astype(np.int32), out_softmax=out_soft.numpy(),
                        weights_sigmoid=wsig.numpy(), ids_sigmoid=isig.numpy().astype(np.int32), vals_sigmoid=vsig.numpy(),
                        out_sigmoid=out_sig.numpy())
    # ---- shared expert (MXFP8)
    g = torch.Generator().manual_seed(21)
    xs = (torch.randn((16, 6144), generator=g) * torch.exp2(torch.randint(-6, 7, (16, 192), generator=g).float()
                                                            ).repeat_interleave(32, 1)).bfloat16()
    xs[0, :64] = 0
    xs[1, :32] = torch.tensor([448.0, 224.0, 0.875, -0.0, 1.0625, 1.1875, 30.0, 31.0] * 4)  # E4M3 ties and the top value
    q8, s8 = ref.shared_mxfp8_quant_ref(xs)
    sw13, ss13, sw2, ss2 = orc.make_shared_weights()
    tsw = [torch.from_numpy(sw13).view(torch.float8_e4m3fn), torch.from_numpy(ss13), torch.from_numpy(sw2).view(torch.float8_e4m3fn),
           torch.from_numpy(ss2)]
    torch_codes = (torch.randn((64, 256), generator=torch.Generator().manual_seed(3)) * 20).to(torch.float8_e4m3fn)
    out_shared = ref.shared_mxfp8_ref(xs, *tsw)
    np.savez_compressed(os.path.join(HERE, "shared.npz"), x_bits=bits(xs), codes=q8.numpy(), scales=s8.numpy(),
                        out=out_shared.numpy(), weight_crc=np.array([zlib.crc32(a.tobytes()) for a in (sw13, ss13, sw2, ss2)],
                                                                    dtype=np.uint32),
                        cast_in=(torch.randn((64, 256), generator=torch.Generator().manual_seed(3)) * 20).numpy(),
                        cast_codes=torch_codes.view(torch.uint8).numpy())
    # ---- sidecar (compact prepared input): FP4 codes rebuilt from the shared FP8 codes + a correction mask
    g = torch.Generator().manual_seed(33)
    xc = (torch.randn((24, 6144), generator=g) * torch.exp2(torch.randint(-8, 9, (24, 192), generator=g).float()
                                                            ).repeat_interleave(32, 1)).bfloat16()
    xc[0, :64] = 0
    xc[1, :32] = torch.tensor([0.75, 1.75, 3.5, -0.75, 0.25, 1.25, 2.5, 5.0, -0.0, 6.0, 0.5, 3.0, 448.0, -3.5, 1.0, 7.0] * 2)
    xc[2, :32] = torch.tensor([0.75, 1.75, 3.5, -0.75, 0.25, 1.25, 2.5, 5.0] * 4) * 0.0078125
    q4, s4 = ref.mxfp4_quant_ref(xc)
    q8c, s8c = ref.shared_mxfp8_quant_ref(xc)
    mask = ref.mxfp4_sidecar_pack_ref(q4, s4, q8c.view(torch.uint8), s8c)
    back = ref.mxfp4_sidecar_unpack_ref(mask, s4, q8c.view(torch.uint8), s8c)
    assert torch.equal(back, q4)
    np.savez_compressed(os.path.join(HERE, "sidecar.npz"), x_bits=bits(xc), q4=q4.numpy(), s4=s4.numpy(),
                        q8=q8c.view(torch.uint8).numpy(), s8=s8c.numpy(), mask=mask.numpy())
    # ---- fused tail: slot sum + shared, residual add, Gemma RMSNorm, MXFP8 of the fp32 norm
    norm = load_norm_reference(root)
    g = torch.Generator().manual_seed(44)
    m = 6
    slots = (torch.randn((m, 4, 6144), generator=g) * torch.exp2(torch.randint(-6, 4, (m, 4, 1), generator=g).float())).bfloat16()
    shared = torch.randn((m, 6144), generator=g).bfloat16()
    resid = (torch.randn((m, 6144), generator=g) * 2.0).bfloat16()
    weight = (torch.randn((6144,), generator=g) * 0.1).bfloat16()
    slots[0, :, :64] = -0.0   # a run of signed zeros through the whole tail
    shared[0, :64] = -0.0
    resid[0, :32] = -0.0
    resid[1, :64] = -slots[1, :, :64].float().sum(0).bfloat16()   # small sums next to cancellation
    slots[2] *= 2.0 ** -20    # a quiet row: tiny rms, eps matters
    shared[2] *= 2.0 ** -20
    resid[2] *= 2.0 ** -20
    x = norm.slots4_local_reference(slots, shared)
    x_noshared = norm.slots4_local_reference(slots, torch.zeros_like(shared))
    y64, res_out = norm.add_rmsnorm_reference(x, resid, weight, 1e-6)
    sb = norm.mxfp8_scale_reference(y64)
    codes = norm.mxfp8_codes(y64, sb)
    np.savez_compressed(os.path.join(HERE, "tail.npz"), slots=bits(slots), shared=bits(shared), residual=bits(resid),
                        weight=bits(weight), eps=np.float32(1e-6), x=bits(x), y64=y64.numpy(), residual_out=bits(res_out),
                        scales=sb.numpy(), codes=codes.numpy(), out=bits(y64.float().bfloat16()))
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
