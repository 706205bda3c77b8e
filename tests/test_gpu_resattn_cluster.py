"""The cluster reducer of ResAttn decode (the KV splits of a sequence and KV head as one thread-block cluster, combined
through distributed shared memory -- "cga_sharded" in the reference's plans, csrc/resattn/plan.py:36-92) against
the ticket reducer: both combine the same partials in split order with the same arithmetic, so the outputs must be
identical bit for bit, and the ticket reducer is the one the oracle tests cover.  Cases include sequences too short
for the later splits (those CTAs leave early and still take part in the cluster), an empty sequence, both head
dimensions, both V / P formats and split counts that are not powers of two."""
import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu


def _inputs(dev, d, page, lens, hkv, g, seed):
    kv = O.make_paged_kv(lens, hkv, d, page, seed=seed)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)   # noqa: E731
    q_np = O.bf16_round(np.random.default_rng(seed).standard_normal((len(lens), hkv * g, d)).astype(np.float32))
    args = (t(q_np).to(torch.bfloat16), t(kv["k_data"]), t(kv["k_sf"]), t(kv["v_data"]), t(kv["v_sf"]),
            t(np.maximum(kv["block_tables"], 0)), t(kv["seq_lens"]), d ** -0.5 * kv["k_global_scale"], kv["v_global_scale"])
    return kv, q_np, args


@pytest.mark.parametrize("d,page,lens,hkv,g,splits,fmt", [
    (128, 16, [3000, 40, 1300], 2, 8, 4, "fp16"),        # the second sequence has one tile: three of its CTAs leave early
    (128, 128, [9000, 513], 8, 8, 8, "fp16"),
    (128, 16, [0, 2500], 1, 4, 2, "fp16"),               # an empty sequence
    (256, 32, [4100, 700], 2, 8, 8, "fp16"),
    (256, 128, [2049], 1, 6, 3, "fp16"),                 # three and five CTAs per cluster
    (128, 64, [6000, 6000, 77], 4, 8, 5, "e4m3"),
    (128, 16, [12000], 8, 8, 7, "fp16"),
    (128, 128, [30000], 8, 8, 16, "fp16"),               # sixteen CTAs: a non-portable cluster size
    (256, 16, [5000, 26000], 2, 4, 16, "fp16"),
])
def test_cluster_reducer_equals_ticket_reducer(cuda_device, device_rcp, d, page, lens, hkv, g, splits, fmt):
    from resinfer_b200 import ops
    dev = cuda_device
    kv, q_np, args = _inputs(dev, d, page, lens, hkv, g, seed=d + splits)
    b, hq = len(lens), hkv * g
    for dtype in (torch.bfloat16, torch.float32):
        outs = {}
        for reducer in ("ticket", "cluster"):
            out = torch.full((b, hq, d), float("nan"), dtype=dtype, device=dev)
            with ops.resattn_pv_format(fmt):
                ops.resattn_decode(*args, out, splits=splits, reducer=reducer, max_kv_len=max(lens))
                ops.resattn_decode(*args, out, splits=splits, reducer=reducer, max_kv_len=max(lens))   # back to back
            torch.cuda.synchronize()
            ops.check_status(dev)
            outs[reducer] = out
        assert not torch.isnan(outs["cluster"]).any()
        assert torch.equal(outs["cluster"], outs["ticket"])
    if fmt == "fp16":
        ref = O.resattn_decode_reference(q_np, kv, d ** -0.5, rcp=O.RecordingRcp(device_rcp))
        got = outs["cluster"].double().cpu().numpy()
        assert np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30) < 3e-3


def test_cluster_reducer_through_the_host_plan(cuda_device):
    from resinfer_b200.nvfp4.cute_attn import host
    from resinfer_b200.nvfp4.cute_attn.kv_layout import NvFp4PagedKVPool
    dev = cuda_device
    d, page, hkv, g, lens = 128, 128, 2, 8, [5000, 2000]
    kv, _, args = _inputs(dev, d, page, lens, hkv, g, seed=1)
    q, kd, ks, vd, vs, bt, sl, score, vscale = args
    pool = NvFp4PagedKVPool(hkv, d, kd, vd, ks, vs, page_size=page, k_global_scale=kv["k_global_scale"],
                            v_global_scale=kv["v_global_scale"])
    outs = []
    for plan in ((4, "kernel"), (4, "cga_sharded")):
        out = torch.zeros(len(lens), hkv * g, d, dtype=torch.bfloat16, device=dev)
        host.run_paged_fp4_decode_qmul4_tmem(q, pool, vd, vs, bt, sl, score, out=out, max_seq_len=max(lens),
                                             value_scale=vscale, plan=plan)
        outs.append(out)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])


def test_cluster_reducer_refuses_what_it_cannot_do(cuda_device):
    from resinfer_b200 import ops
    dev = cuda_device
    _, _, args = _inputs(dev, 128, 16, [600], 1, 8, seed=2)
    out = torch.zeros(1, 8, 128, dtype=torch.bfloat16, device=dev)
    for splits in (1, 9, 12, 32):
        with pytest.raises(RuntimeError, match="cluster reducer takes 2 to 8 or 16 splits"):
            ops.resattn_decode(*args, out, splits=splits, reducer="cluster")
    packed = torch.zeros(1, 8 * 64, dtype=torch.uint8, device=dev)
    with pytest.raises(RuntimeError, match="cluster reducer"):
        ops.resattn_decode(*args, packed, splits=2, reducer="cluster",
                           out_global_scale=torch.ones(1, device=dev),
                           out_block_scale=torch.zeros(128 * 64, dtype=torch.uint8, device=dev))
    with pytest.raises(KeyError):
        ops.resattn_decode(*args, out, splits=2, reducer="dsmem")
