"""Generates the golden fixtures of this directory.  Run on a B200 box, from the repository root:

    python oracle/build_ref.py            # on a machine that has the reference checkout
    python tests/golden/make_golden.py    # on the GPU box; writes tests/golden/*.npz

Every fixture holds the outputs of the REFERENCE project's own CUDA quantiser kernels
(``oracle/_ref/libnvfp4_ref.so``, compiled from the reference sources) on small seeded inputs,
the inputs themselves (bf16 bit patterns) and the device's rcp.approx.ftz.f32 results for the
reciprocals the algorithm takes on those inputs, so that the CPU oracle can be checked bit for bit
without a GPU.  ``case`` strings encode the parameters.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

import oracle as O  # noqa: E402
from resinfer_b200 import nvfp4, ops  # noqa: E402

OUT = os.environ.get("GOLDEN_OUT", HERE)


def main():
    dev = torch.device("cuda", 0)
    nvfp4.ensure_loaded()
    torch.ops.load_library(os.path.join(ROOT, "oracle", "_ref", "libnvfp4_ref.so"))
    ref = torch.ops.nvfp4_ref

    def dev_rcp(x):
        return ops.rcp_approx(torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(dev)).cpu().numpy()

    def to_dev(x_np):
        return torch.from_numpy(x_np).to(torch.bfloat16).to(dev)

    def save(name, rec, **arrays):
        k, v = rec.table()
        np.savez_compressed(os.path.join(OUT, name + ".npz"), rcp_keys=k, rcp_vals=v, **arrays)
        print("wrote", name, {a: arrays[a].shape for a in arrays})

    # ---- NVFP4 MEXT, five layouts (+ one dual-scale case) -----------------------------------
    for (m, k, seed) in [(1, 256, 11), (5, 512, 12), (16, 1024, 13)]:
        x_np = O.make_activation(m, k, seed=seed)
        x = to_dev(x_np)
        gs_inv = np.float32(6 * 448) / np.float32(np.abs(x_np).max())
        for layout in range(5):
            for dual in ((False, True) if (layout == 1 and m == 5) else (False,)):
                gi = [gs_inv, gs_inv * np.float32(3.0)] if dual else [gs_inv]
                gi_t = torch.tensor(gi, dtype=torch.float32, device=dev)
                out_m = (m + 7) // 8 * 8 if layout in (2, 4) else m
                oc, osf, wr = O.nvfp4_quant_mext(x_np, gi[0], layout, gs_inv_res=gi[1] if dual else None,
                                                 rcp=(rec := O.RecordingRcp(dev_rcp)))
                codes = torch.zeros(out_m * k, dtype=torch.uint8, device=dev)
                sf = torch.zeros(osf.size, dtype=torch.uint8, device=dev)
                ref.scaled_fp4_quant_mext_r1(codes, x, sf, gi_t, 0, layout, False)
                save(f"nvfp4_mext_m{m}_k{k}_L{layout}{'_dual' if dual else ''}", rec,
                     x_bits=O.to_bf16_bits(x_np), gs_inv=np.array(gi, np.float32), layout=np.int32(layout),
                     codes=codes.cpu().numpy().reshape(oc.shape), sf=sf.cpu().numpy(), sf_written=wr)
    # ---- NVFP4 KEXT ---------------------------------------------------------------------------
    for (m, k, seed) in [(3, 256, 21), (9, 512, 22)]:
        x_np = O.make_activation(m, k, seed=seed)
        x = to_dev(x_np)
        gs_inv = np.float32(6 * 448) / np.float32(np.abs(x_np).max())
        gi_t = torch.tensor([gs_inv], dtype=torch.float32, device=dev)
        for per8 in (1, 2, 4):
            mask = O.make_kext_mask(k, per8, seed=per8)
            s = k // 8 * per8
            oc, osf, wr = O.nvfp4_quant_kext(x_np, gs_inv, mask, per8, rcp=(rec := O.RecordingRcp(dev_rcp)))
            codes = torch.zeros(m * (k + s) // 2, dtype=torch.uint8, device=dev)
            sf = torch.zeros(osf.size, dtype=torch.uint8, device=dev)
            ref.scaled_fp4_quant(codes, x, sf, gi_t, torch.from_numpy(mask).to(dev), k + s, per8, False)
            save(f"nvfp4_kext_m{m}_k{k}_p{per8}", rec, x_bits=O.to_bf16_bits(x_np), gs_inv=np.array([gs_inv], np.float32),
                 mask=mask, per8=np.int32(per8), codes=codes.cpu().numpy().reshape(oc.shape), sf=sf.cpu().numpy(),
                 sf_written=wr)
    # ---- MXFP4 MEXT / selective ---------------------------------------------------------------
    for (m, k, seed) in [(5, 256, 31), (12, 384, 32)]:
        x_np = O.make_activation(m, k, seed=seed)
        x = to_dev(x_np)
        for tile8, swz in ((False, True), (True, True), (False, False)):
            oc, osf = O.mxfp4_quant_mext(x_np, swizzle=swz, tile8=tile8, m_pad_multiple=8 if tile8 else None,
                                         rcp=(rec := O.RecordingRcp(dev_rcp)))
            codes = torch.full(oc.shape, 0x55, dtype=torch.uint8, device=dev)
            sf = torch.full(osf.shape, 0x55, dtype=torch.uint8, device=dev)
            ref.mxfp4_residue_quant(x, codes, sf, None, 0, swz, tile8, 0)
            save(f"mxfp4_mext_m{m}_k{k}_{'tile8' if tile8 else 'pair'}_{'sw' if swz else 'lin'}", rec,
                 x_bits=O.to_bf16_bits(x_np), tile8=np.int32(tile8), swizzle=np.int32(swz), codes=codes.cpu().numpy(),
                 sf=sf.cpu().numpy())
        for per8 in (1, 2, 4):
            mask = O.make_kext_mask(k, per8, seed=per8)
            oc, osf = O.mxfp4_quant_selective(x_np, mask, per8, rcp=(rec := O.RecordingRcp(dev_rcp)))
            codes = torch.full(oc.shape, 0x55, dtype=torch.uint8, device=dev)
            sf = torch.full(osf.shape, 0x55, dtype=torch.uint8, device=dev)
            ref.mxfp4_residue_quant(x, codes, sf, torch.from_numpy(mask).to(dev), per8, True, False, 0)
            save(f"mxfp4_sel_m{m}_k{k}_p{per8}", rec, x_bits=O.to_bf16_bits(x_np), mask=mask, per8=np.int32(per8),
                 codes=codes.cpu().numpy(), sf=sf.cpu().numpy())
    # ---- grouped query quantiser ----------------------------------------------------------------
    for (b, h, g, d, seed) in [(2, 2, 8, 128, 41), (1, 1, 4, 128, 42), (1, 2, 6, 256, 43)]:
        q_np = O.bf16_round(np.random.default_rng(seed).standard_normal((b, h, g, d)).astype(np.float32))
        p = 8 if g == 4 else 16
        op, osf = O.nvfp4_quant_grouped_q(q_np, rcp=(rec := O.RecordingRcp(dev_rcp)))
        qp = torch.zeros(b, h, p, d // 2, dtype=torch.uint8, device=dev)
        qs = torch.zeros(osf.size, dtype=torch.uint8, device=dev)
        ref.scaled_fp4_quant_mext_r1_grouped_q(to_dev(q_np), qp, qs)
        save(f"grouped_q_b{b}_h{h}_g{g}_d{d}", rec, q_bits=O.to_bf16_bits(q_np), q_pack=qp.cpu().numpy(),
             q_sf=qs.cpu().numpy())
    torch.cuda.synchronize()


if __name__ == "__main__":
    main()
