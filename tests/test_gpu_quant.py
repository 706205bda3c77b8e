"""GPU parity of the quantiser kernels, called through the reference-named ops (C ABI underneath):
bit-exact against (a) the reference project's own compiled kernels when oracle/_ref is present,
(b) the CPU oracle fed with the device's rcp.approx results, (c) the committed golden fixtures."""
import glob
import os

import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu
GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


def _bf16(x, dev):
    return torch.from_numpy(x).to(torch.bfloat16).to(dev)


def _eq(a, b, mask=None):
    a = a.cpu().numpy().ravel() if hasattr(a, "cpu") else np.asarray(a).ravel()
    b = b.cpu().numpy().ravel() if hasattr(b, "cpu") else np.asarray(b).ravel()
    if mask is not None:
        a, b = a[mask.ravel()], b[mask.ravel()]
    assert a.shape == b.shape
    bad = int((a != b).sum())
    assert bad == 0, f"{bad} of {a.size} bytes differ"


@pytest.mark.parametrize("m,k", [(1, 256), (7, 512), (16, 5120), (128, 2048), (130, 1024), (33, 8192)])
@pytest.mark.parametrize("layout", range(5))
def test_nvfp4_mext(cuda_device, device_rcp, ref_ops, m, k, layout):
    from resinfer_b200 import nvfp4
    x_np = O.make_activation(m, k, seed=m + k)
    x = _bf16(x_np, cuda_device)
    gi_np = np.float32(6 * 448) / np.float32(np.abs(x_np).max())
    gi = torch.tensor([gi_np], dtype=torch.float32, device=cuda_device)
    kw = {"m_pad_multiple": 8} if layout in (2, 4) else {}
    codes, sf = nvfp4.scaled_fp4_quant_mext_r1(x, gi, layout_mode=layout, **kw)
    oc, osf, wr = O.nvfp4_quant_mext(x_np, gi_np, layout, rcp=O.RecordingRcp(device_rcp))
    _eq(codes, oc)
    _eq(sf, osf, wr)
    if ref_ops is not None:
        rc = torch.empty_like(codes)
        rs = torch.zeros_like(sf)
        ref_ops.scaled_fp4_quant_mext_r1(rc.view(-1), x, rs, gi, 0, layout, False)
        _eq(codes, rc)
        _eq(sf, rs, wr)


def test_nvfp4_mext_dual_scale_fp16_and_strided_input(cuda_device, device_rcp, ref_ops):
    from resinfer_b200 import nvfp4
    m, k = 9, 512
    x_np = O.make_activation(m, k, seed=3)
    gi = torch.tensor([40.0, 900.0], dtype=torch.float32, device=cuda_device)
    x = _bf16(x_np, cuda_device)
    codes, sf = nvfp4.scaled_fp4_quant_mext_r1(x, gi, layout_mode="row_pair")
    oc, osf, wr = O.nvfp4_quant_mext(x_np, np.float32(40.0), 1, gs_inv_res=np.float32(900.0), rcp=O.RecordingRcp(device_rcp))
    _eq(codes, oc)
    _eq(sf, osf, wr)
    # fp16 input
    xh_np = x_np.astype(np.float16).astype(np.float32)
    xh = torch.from_numpy(xh_np).to(torch.float16).to(cuda_device)
    codes, sf = nvfp4.scaled_fp4_quant_mext_r1(xh, gi[:1], layout_mode="concat_k")
    oc, osf, wr = O.nvfp4_quant_mext(xh_np, np.float32(40.0), 3, rcp=O.RecordingRcp(device_rcp))
    _eq(codes, oc)
    _eq(sf, osf, wr)
    if ref_ops is not None:
        rc, rs = torch.empty_like(codes), torch.zeros_like(sf)
        ref_ops.scaled_fp4_quant_mext_r1(rc.view(-1), xh, rs, gi[:1], 0, 3, False)
        _eq(codes, rc)
    # a row-strided view (K slice of a wider tensor), as a row-parallel shard sees it
    wide = _bf16(O.make_activation(m, 2 * k, seed=4), cuda_device)
    view = wide[:, k:]
    c1, s1 = nvfp4.scaled_fp4_quant_mext_r1(view, gi[:1], layout_mode=1)
    c2, s2 = nvfp4.scaled_fp4_quant_mext_r1(view.contiguous(), gi[:1], layout_mode=1)
    _eq(c1, c2)


@pytest.mark.parametrize("m,k", [(1, 256), (16, 5120), (130, 1024), (20, 25600)])
@pytest.mark.parametrize("per8", [1, 2, 4])
def test_nvfp4_kext(cuda_device, device_rcp, ref_ops, m, k, per8):
    from resinfer_b200 import nvfp4
    x_np = O.make_activation(m, k, seed=m + k + per8)
    x = _bf16(x_np, cuda_device)
    gi_np = np.float32(6 * 448) / np.float32(np.abs(x_np).max())
    gi = torch.tensor([gi_np], dtype=torch.float32, device=cuda_device)
    mask_np = O.make_kext_mask(k, per8, seed=per8)
    s = k // 8 * per8
    codes, sf = nvfp4.scaled_fp4_quant_with_mask(x, gi, torch.from_numpy(mask_np).to(cuda_device), s)
    oc, osf, wr = O.nvfp4_quant_kext(x_np, gi_np, mask_np, per8, rcp=O.RecordingRcp(device_rcp))
    _eq(codes, oc)
    _eq(sf, osf, wr)
    # the index-based entry builds the same mask
    idx = torch.from_numpy(O.mask_to_indices(mask_np)).to(cuda_device)
    c2, s2 = nvfp4.scaled_fp4_quant(x, gi, idx)
    _eq(c2, codes)
    if ref_ops is not None:
        rc, rs = torch.empty_like(codes), torch.zeros_like(sf)
        ref_ops.scaled_fp4_quant(rc.view(-1), x, rs, gi, torch.from_numpy(mask_np).to(cuda_device), k + s, per8, False)
        _eq(codes, rc)
        _eq(sf, rs, wr)


def test_kext_ratio_one_is_rejected(cuda_device):
    x = torch.zeros(4, 256, dtype=torch.bfloat16, device=cuda_device)
    out = torch.empty(4 * 256, dtype=torch.uint8, device=cuda_device)
    sf = torch.empty(8 * 512, dtype=torch.uint8, device=cuda_device)
    with pytest.raises(RuntimeError, match="no longer supported"):
        torch.ops.nvfp4.scaled_fp4_quant(out, x, sf, torch.ones(1, device=cuda_device),
                                         torch.full((32,), 255, dtype=torch.uint8, device=cuda_device), 512, 8, False)
    with pytest.raises(RuntimeError, match="too small"):
        torch.ops.nvfp4.scaled_fp4_quant_mext_r1(out[:16], x, sf, torch.ones(1, device=cuda_device), 0, 1, True)


@pytest.mark.parametrize("m,k", [(1, 256), (7, 512), (16, 5120), (130, 1024), (64, 8192)])
def test_mxfp4_mext_and_selective(cuda_device, device_rcp, ref_ops, m, k):
    from resinfer_b200.nvfp4 import mxfp4 as mx
    x_np = O.make_activation(m, k, seed=m + k)
    x = _bf16(x_np, cuda_device)
    for tile8, layout in ((False, "128x4"), (True, "128x4"), (False, "linear")):
        kw = dict(mext_layout="tile8", m_pad_multiple=8) if tile8 else {}
        codes, sf = mx.quantize_mext(x, layout=layout, **kw)
        oc, osf = O.mxfp4_quant_mext(x_np, swizzle=layout == "128x4", tile8=tile8, m_pad_multiple=8 if tile8 else None,
                                     rcp=O.RecordingRcp(device_rcp))
        _eq(codes, oc)
        _eq(sf, osf)
        if ref_ops is not None:
            rc, rs = torch.full_like(codes, 0x55), torch.full_like(sf, 0x55)
            ref_ops.mxfp4_residue_quant(x, rc, rs, None, 0, layout == "128x4", tile8, 0)
            _eq(codes, rc)
            _eq(sf, rs)
    for per8 in (1, 2, 4):
        mask_np = O.make_kext_mask(k, per8, seed=per8)
        idx, mask = mx.prepare_indices(O.mask_to_indices(mask_np).tolist(), k, cuda_device)
        codes, sf = mx.quantize_selective(x, idx, mask)
        oc, osf = O.mxfp4_quant_selective(x_np, mask_np, per8, rcp=O.RecordingRcp(device_rcp))
        _eq(codes, oc)
        _eq(sf, osf)
        if ref_ops is not None:
            rc, rs = torch.full_like(codes, 0x55), torch.full_like(sf, 0x55)
            ref_ops.mxfp4_residue_quant(x, rc, rs, mask, per8, True, False, 0)
            _eq(codes, rc)
            _eq(sf, rs)
    # plain quantisation = the base rows of the MEXT output
    pc, ps = mx.quantize(x)
    oc, osf = O.mxfp4_quant_plain(x_np, rcp=O.RecordingRcp(device_rcp))
    _eq(pc, oc)
    _eq(ps, osf)
    assert mx.quantize(x[:0])[0].shape == (0, k // 2)


@pytest.mark.parametrize("b,h,g,d", [(2, 2, 8, 128), (1, 3, 4, 128), (2, 1, 6, 256), (5, 8, 8, 256)])
def test_grouped_q(cuda_device, device_rcp, ref_ops, b, h, g, d):
    q_np = O.bf16_round(np.random.default_rng(b + d).standard_normal((b, h, g, d)).astype(np.float32))
    q = _bf16(q_np, cuda_device)
    p = 8 if g == 4 else 16
    qp = torch.zeros(b, h, p, d // 2, dtype=torch.uint8, device=cuda_device)
    qs = torch.zeros(b * h * 128 * d // 16, dtype=torch.uint8, device=cuda_device)
    torch.ops.nvfp4.scaled_fp4_quant_mext_r1_grouped_q(q, qp, qs)
    op, osf = O.nvfp4_quant_grouped_q(q_np, rcp=O.RecordingRcp(device_rcp))
    _eq(qp, op)
    _eq(qs, osf)
    if ref_ops is not None:
        rp, rs = torch.zeros_like(qp), torch.zeros_like(qs)
        ref_ops.scaled_fp4_quant_mext_r1_grouped_q(q, rp, rs)
        _eq(qp, rp)
        _eq(qs, rs)
    with pytest.raises(RuntimeError, match="GQA4/6/8"):
        torch.ops.nvfp4.scaled_fp4_quant_mext_r1_grouped_q(q[:, :, :3].contiguous(), qp, qs)


@pytest.mark.parametrize("path", GOLDEN, ids=os.path.basename)
def test_kernels_reproduce_golden_fixtures(cuda_device, path):
    """Our kernels against the stored outputs of the reference kernels (works without oracle/_ref)."""
    from resinfer_b200 import nvfp4
    from resinfer_b200.nvfp4 import mxfp4 as mx
    z = np.load(path)
    name = os.path.basename(path)
    if name.startswith("grouped_q"):
        q_np = O.from_bf16_bits(z["q_bits"])
        q = _bf16(q_np, cuda_device)
        qp, qs = torch.zeros(z["q_pack"].shape, dtype=torch.uint8, device=cuda_device), torch.zeros(
            z["q_sf"].shape, dtype=torch.uint8, device=cuda_device)
        torch.ops.nvfp4.scaled_fp4_quant_mext_r1_grouped_q(q, qp, qs)
        _eq(qp, z["q_pack"])
        _eq(qs, z["q_sf"])
        return
    x_np = O.from_bf16_bits(z["x_bits"])
    x = _bf16(x_np, cuda_device)
    if name.startswith("nvfp4_mext"):
        layout = int(z["layout"])
        gi = torch.from_numpy(z["gs_inv"]).to(cuda_device)
        kw = {"m_pad_multiple": 8} if layout in (2, 4) else {}
        codes, sf = nvfp4.scaled_fp4_quant_mext_r1(x, gi, layout_mode=layout, **kw)
        _eq(codes, z["codes"])
        _eq(sf, z["sf"], z["sf_written"])
    elif name.startswith("nvfp4_kext"):
        per8 = int(z["per8"])
        codes, sf = nvfp4.scaled_fp4_quant_with_mask(x, torch.from_numpy(z["gs_inv"]).to(cuda_device),
                                                     torch.from_numpy(z["mask"]).to(cuda_device), x.shape[1] // 8 * per8)
        _eq(codes, z["codes"])
        _eq(sf, z["sf"], z["sf_written"])
    elif name.startswith("mxfp4_mext"):
        t8 = bool(z["tile8"])
        kw = dict(mext_layout="tile8", m_pad_multiple=8) if t8 else {}
        codes, sf = mx.quantize_mext(x, layout="128x4" if bool(z["swizzle"]) else "linear", **kw)
        _eq(codes, z["codes"])
        _eq(sf, z["sf"])
    else:
        per8 = int(z["per8"])
        idx, mask = mx.prepare_indices(O.mask_to_indices(z["mask"]).tolist(), x.shape[1], cuda_device)
        codes, sf = mx.quantize_selective(x, idx, mask)
        _eq(codes, z["codes"])
        _eq(sf, z["sf"])


def test_quantiser_roundtrip_property_at_full_size(cuda_device):
    """Size-independent property on a benchmark-sized input (down projection, M=128): dequantised base +
    dequantised residue reconstructs x far better than the base alone, for every row."""
    from resinfer_b200 import nvfp4
    m, k = 128, 25600
    g = torch.Generator(device=cuda_device).manual_seed(0)
    x = torch.randn(m, k, generator=g, device=cuda_device).to(torch.bfloat16)
    gs = float(x.float().abs().max()) / (6 * 448)
    gi = torch.tensor([1 / gs], dtype=torch.float32, device=cuda_device)
    codes, sf = nvfp4.scaled_fp4_quant_mext_r1(x, gi, layout_mode=1)
    a = O.dequant_operand(codes.cpu().numpy(), sf.cpu().numpy(), "nvfp4") * np.float32(gs)
    xr = x.float().cpu().numpy()
    e0 = np.linalg.norm(xr - a[0::2], axis=1)
    e1 = np.linalg.norm(xr - a[0::2] - a[1::2], axis=1)
    assert np.all(e1 < 0.3 * e0)
    # concat_k holds the same codes as row_pair
    ck, _ = nvfp4.scaled_fp4_quant_mext_r1(x, gi, layout_mode=3)
    assert torch.equal(ck[:, :k // 2], codes[0::2]) and torch.equal(ck[:, k // 2:], codes[1::2])
