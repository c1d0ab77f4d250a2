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
        if "ipcfail" in mask:  # host-side fault injection: rank 1 reports that it could not map its peers' buffers
            os.environ["RA_FAULT_IPC_OPEN"] = "1"
        dtype = getattr(torch, dtype)
        nb = 1 if "b1" in mask else 2  # one batch element: the backward splits its own block by heads, or not at all
        q, k, v, do, rng = make_inputs(5, nb, lq, lk, h, d, dtype)
        seg = rng.integers(0, 3, (nb, max(lq, lk))).astype(np.int32)
        import re

        cq, ck = lq // world, lk // world

        def shard_of(r):
            if "zigzag" in mask:  # rank r holds chunks r and 2N-1-r; positions say where each token is
                return ra.zigzag_indices(lq, r, world).numpy(), ra.zigzag_indices(lk, r, world).numpy()
            return np.arange(r * cq, (r + 1) * cq), np.arange(r * ck, (r + 1) * ck)

        sq, sk = shard_of(rank)
        window = int(re.search(r"window(\d+)", mask).group(1)) if "window" in mask else 0
        qpos = np.broadcast_to(np.arange(lq, dtype=np.int32), (nb, lq))
        kpos = np.broadcast_to(np.arange(lk, dtype=np.int32), (nb, lk))
        bias, fn, qkw, kkw = None, None, None, None
        if mask != "none":
            use_seg = "seg" in mask
            bias = O.score_mod_bias(nb, h, qpos, kpos, seg[:, :lq] if use_seg else None, seg[:, :lk] if use_seg else None,
                                    causal="causal" in mask, window=window)
            fn = ra.ScoreMod(causal="causal" in mask, window=window)
            T = lambda a: to_dev(a, torch.int32)
            qkw = {"q_positions": T(qpos[:, sq]), "q_segment_ids": T(seg[:, :lq][:, sq]) if use_seg else None}
            kkw = {"kv_positions": T(kpos[:, sk]), "kv_segment_ids": T(seg[:, :lk][:, sk]) if use_seg else None}
        if mask == "callable":
            pass
        with ra.Mesh((1, world), ("dp", "sp")) as mesh:
            # every rank ends up on the same transport; one rank that cannot map moves the whole ring to NCCL
            want_transport = "nccl" if ("nccl" in mask or "ipcfail" in mask) else "p2p"
            assert mesh.ring("sp").transport == want_transport, mesh.ring("sp").transport
            tq, tk, tv = (to_dev(x, dtype).requires_grad_(True) for x in (q[:, sq], k[:, sk], v[:, sk]))
            if "reserve" in mask:  # buffers and handle exchange ahead of the first call
                ra.reserve(tq, tk, tv, "sp", bias_kv_kwargs=kkw)
            plan = None
            if "plan" in mask:  # leave out the ring steps whose block the mask empties
                plan = ra.make_ring_plan(tq, tk, "sp", fn, qkw, kkw)
                vis = np.isfinite(bias).any(axis=(0, 1))  # [lq, lk]
                want = [[bool(vis[np.ix_(shard_of(r)[0], shard_of(o)[1])].any()) or r == o for o in range(world)]
                        for r in range(world)]
                got = plan.matrix()
                # the plan works on 128-token summaries: it may keep a pair that is in fact empty, never drop one
                for r in range(world):
                    for o in range(world):
                        assert got[r][o] or not want[r][o], f"plan drops pair ({r}, {o}) that has visible pairs"
                if not all(map(all, want)):
                    assert sum(map(sum, got)) < world * world, "the plan keeps every pair although some are empty"
                # row runs: every key row some query of r sees lies inside a run of the pair (r, o); a
                # window mask needs less than the whole block of its left neighbour
                moved = 0
                for r in range(world):
                    for o in range(world):
                        if r == o or not got[r][o]:
                            continue
                        runs = plan.rows(r, o)
                        inside = np.zeros(ck, bool)
                        for lo, hi in runs:
                            inside[lo:hi] = True
                        seen = vis[np.ix_(shard_of(r)[0], shard_of(o)[1])].any(axis=0)
                        assert not (seen & ~inside).any(), f"pair ({r}, {o}): visible key rows outside the runs {runs}"
                        moved += int(inside.sum())
                if window and window < ck // 2:
                    assert moved < ck * sum(got[r][o] for r in range(world) for o in range(world) if r != o), "no halo"
            for rep in range(2):  # second pass reuses the ring's buffers
                tq.grad = tk.grad = tv.grad = None
                out = ra.ring_attention(tq, tk, tv, "sp", bias_fn=fn, bias_q_kwargs=qkw, bias_kv_kwargs=kkw,
                                        block_impl=impl, plan=plan)
                out.backward(to_dev(do[:, sq], dtype))
            torch.cuda.synchronize()
            # no bounded wait ran out, inside a kernel or for a peer
            assert ra.device_status() == 0 and not mesh.ring("sp").aborted
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
    ("bfloat16", 2048, 2048, 2, 128, "causal+window256+plan", "tcgen05"),
    ("bfloat16", 4096, 4096, 2, 128, "causal+window300+zigzag+plan", "tcgen05"),
    ("float32", 512, 512, 2, 32, "causal+window100+plan+nccl", "simt"),
    ("bfloat16", 2048, 2048, 2, 128, "causal+zigzag+ipcfail", "tcgen05"),
    ("bfloat16", 2048, 2048, 2, 128, "causal+seg+zigzag+reserve", "tcgen05"),
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
