"""Multi-GPU ring tests: one process per GPU over NCCL (skipped with fewer than 2 GPUs).

Each rank holds one contiguous shard; the ring result is compared with dense attention on
the unsharded arrays (the property of ring_attention/ring_test.py:45-300).
"""
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, case, q_out):
    try:
        sys.path.insert(0, ROOT)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        import torch.distributed as dist

        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        import ring_attention_b200 as ra
        from oracle import oracle as O
        from tests.util import check_close, make_inputs, to_dev

        dtype, lq, lk, h, d, mask, impl = case
        if "nccl" in mask:  # the NCCL send/recv transport instead of the default peer copies
            os.environ["RA_TRANSPORT"] = "nccl"
        dtype = getattr(torch, dtype)
        nb = 1 if "b1" in mask else 2  # one batch element: the backward splits its own block by heads, or not at all
        q, k, v, do, rng = make_inputs(5, nb, lq, lk, h, d, dtype)
        seg = rng.integers(0, 3, (nb, max(lq, lk))).astype(np.int32)
        cq, ck = lq // world, lk // world
        sq, sk = slice(rank * cq, (rank + 1) * cq), slice(rank * ck, (rank + 1) * ck)
        if "zigzag" in mask:  # rank r holds chunks r and 2N-1-r; positions say where each token is
            sq = ra.zigzag_indices(lq, rank, world).numpy()
            sk = ra.zigzag_indices(lk, rank, world).numpy()
        qpos = np.broadcast_to(np.arange(lq, dtype=np.int32), (nb, lq))
        kpos = np.broadcast_to(np.arange(lk, dtype=np.int32), (nb, lk))
        bias, fn, qkw, kkw = None, None, None, None
        if mask != "none":
            use_seg = "seg" in mask
            bias = O.score_mod_bias(nb, h, qpos, kpos, seg[:, :lq] if use_seg else None, seg[:, :lk] if use_seg else None,
                                    causal="causal" in mask)
            fn = ra.ScoreMod(causal="causal" in mask)
            T = lambda a: to_dev(a, torch.int32)
            qkw = {"q_positions": T(qpos[:, sq]), "q_segment_ids": T(seg[:, :lq][:, sq]) if use_seg else None}
            kkw = {"kv_positions": T(kpos[:, sk]), "kv_segment_ids": T(seg[:, :lk][:, sk]) if use_seg else None}
        if mask == "callable":
            pass
        with ra.Mesh((1, world), ("dp", "sp")):
            tq, tk, tv = (to_dev(x, dtype).requires_grad_(True) for x in (q[:, sq], k[:, sk], v[:, sk]))
            for rep in range(2):  # second pass reuses the ring's buffers
                tq.grad = tk.grad = tv.grad = None
                out = ra.ring_attention(tq, tk, tv, "sp", bias_fn=fn, bias_q_kwargs=qkw, bias_kv_kwargs=kkw,
                                        block_impl=impl)
                out.backward(to_dev(do[:, sq], dtype))
            torch.cuda.synchronize()
        ref = O.mha(q, k, v, bias)
        rq, rk, rv = O.mha_grads(q, k, v, do, bias)
        check_close(out, ref[:, sq], dtype, "out")
        check_close(tq.grad, rq[:, sq], dtype, "dq", 2e-5)
        check_close(tk.grad, rk[:, sk], dtype, "dk", 2e-5)
        check_close(tv.grad, rv[:, sk], dtype, "dv", 2e-5)
        dist.barrier()
        dist.destroy_process_group()
        q_out.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback

        q_out.put((rank, traceback.format_exc()))


CASES = [
    ("float32", 512, 512, 2, 64, "causal", "simt"),
    ("float32", 256, 512, 2, 32, "none", "simt"),
    ("bfloat16", 1024, 1024, 2, 128, "causal+seg", "cuda"),
    ("bfloat16", 2048, 2048, 2, 128, "causal", "cuda"),
    ("bfloat16", 4096, 4096, 2, 128, "causal+zigzag", "tcgen05"),
    ("bfloat16", 2048, 2048, 2, 64, "causal+seg+zigzag", "tcgen05"),
    ("bfloat16", 2048, 2048, 2, 128, "causal+zigzag+nccl", "tcgen05"),
    ("bfloat16", 2048, 2048, 2, 128, "causal+zigzag+b1", "tcgen05"),
    ("float32", 256, 256, 1, 32, "causal+b1", "simt"),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(str(x) for x in c))
def test_ring_over_nccl(case):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = 29700 + (hash(case) % 200)
    procs = [ctx.Process(target=_worker, args=(r, world, port, case, q_out)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q_out.get(timeout=600) for _ in range(world)]
    for p in procs:
        p.join(120)
    for rank, msg in res:
        assert msg == "ok", f"rank {rank}: {msg}"
