"""Two CPU processes over gloo walk the engine's ring schedule.

The CUDA ring (csrc/ring.cu) cannot run without GPUs, so this test drives the same
schedule -- at step t a rank works on the K/V block of rank `ra_ring_source(rank, N, t)`,
which the owner sends directly; in the backward each step's dK/dV contribution goes
straight back to the owner -- with the oracle's block math and torch.distributed
send/recv, and checks the result against dense attention.
"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _exchange(send_arr, to, frm, do_send=True, do_recv=True):
    """One ring exchange; either half can be left out (both of its ends must agree)."""
    recv = torch.empty_like(send_arr)
    ops = []
    if do_send:
        ops.append(dist.P2POp(dist.isend, send_arr, to))
    if do_recv:
        ops.append(dist.P2POp(dist.irecv, recv, frm))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    return recv if do_recv else None


def _worker(rank, world, port, q_out, window=0, plan=False):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as O
    from ring_attention_b200 import Mesh
    from ring_attention_b200._lib import lib

    assert Mesh.axis_ranks(rank, 1, (1, world)) == list(range(world))
    rng = np.random.default_rng(0)
    b, S, h, d = 2, 48, 2, 8
    q, k, v, do = (rng.standard_normal((b, S, h, d)) for _ in range(4))
    pos = np.broadcast_to(np.arange(S), (b, S))
    c = S // world
    sl = slice(rank * c, (rank + 1) * c)
    bh = lambda x: np.ascontiguousarray(np.transpose(x[:, sl], (0, 2, 1, 3)))
    ql, kl, vl, dol = bh(q), bh(k), bh(v), bh(do)
    qpos, kpos = pos[:, sl], np.ascontiguousarray(pos[:, sl])
    scale = 1 / np.sqrt(d)
    o = np.zeros_like(ql)
    m = np.full(ql.shape[:3], -np.inf)
    l = np.zeros(ql.shape[:3])

    def mask_bias(qp, kp):
        return O.score_mod_bias(b, 1, qp, kp, None, None, causal=True, window=window)

    bias_full = mask_bias(pos, pos)
    # The plan of the CUDA schedule: need[r][o] says whether the queries of rank r see anything in
    # the block of rank o.  Every rank holds the same matrix, so the two ends of a transfer agree.
    vis = np.isfinite(bias_full).any(axis=(0, 1))
    need = [[(not plan) or r == o_ or bool(vis[r * c:(r + 1) * c, o_ * c:(o_ + 1) * c].any()) for o_ in range(world)]
            for r in range(world)]
    if plan:
        assert not all(map(all, need)), "this mask should empty at least one pair"
    blocks = []
    for t in range(world):
        src = lib.ra_ring_source(rank, world, t)
        if t == 0:
            kt, vt, pt = kl, vl, kpos
        else:  # the owner sends straight to its consumer
            to, frm = (rank + t) % world, (rank - t) % world
            assert frm == src
            snd, rcv = need[to][rank], need[rank][frm]
            kt, vt, pt = (_exchange(torch.from_numpy(x), to, frm, snd, rcv) for x in (kl, vl, kpos))
            if not rcv:  # nothing visible in this block: no wait, no block update
                blocks.append(None)
                continue
            kt, vt, pt = kt.numpy(), vt.numpy(), pt.numpy()
        bias = mask_bias(qpos, pt)
        o, m, l = O.fwd_block(ql, kt, vt, bias, o, m, l, scale)
        blocks.append((kt, vt, bias))
    out, L = O.finalize(o, m, l)
    dq = np.zeros_like(ql)
    dk = np.zeros_like(kl)
    dv = np.zeros_like(vl)
    for t in range(world):
        owner, giver = (rank - t) % world, (rank + t) % world
        compute, receive = blocks[t] is not None, need[giver][rank]
        dk_ = dv_ = np.zeros_like(kl)
        if compute:
            kt, vt, bias = blocks[t]
            dq_, dk_, dv_ = O.bwd_block(ql, kt, vt, bias, out, L, dol, scale)
            dq += dq_
        if t == 0:
            dk += dk_
            dv += dv_
        else:  # contribution goes to the owner (rank - t), ours comes from rank + t
            got = [_exchange(torch.from_numpy(np.ascontiguousarray(x)), owner, giver, compute, receive) for x in (dk_, dv_)]
            if receive:
                dk += got[0].numpy()
                dv += got[1].numpy()
    ref = O.mha(q, k, v, bias_full)
    rq, rk, rv = O.mha_grads(q, k, v, do, bias_full)
    un = lambda x: np.transpose(x, (0, 2, 1, 3))
    err = max(
        np.abs(un(out) - ref[:, sl]).max(), np.abs(un(dq) - rq[:, sl]).max(),
        np.abs(un(dk) - rk[:, sl]).max(), np.abs(un(dv) - rv[:, sl]).max(),
    )
    q_out.put((rank, float(err)))
    dist.destroy_process_group()


@pytest.mark.parametrize("world,window,plan", [(2, 0, False), (3, 0, False), (3, 10, True), (2, 5, True)])
def test_direct_ring_schedule_over_gloo(world, window, plan):
    """Without a plan every step runs; with one, the transfers and block updates of the pairs the
    window mask empties are left out, each end deciding from the same matrix."""
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = 29600 + world + 10 * int(plan) + (window % 7)
    procs = [ctx.Process(target=_worker, args=(r, world, port, q_out, window, plan)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q_out.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, err in res:
        assert err < 1e-12, (rank, err)
