"""CPU tests of the multi-GPU host logic: view partitioning, buffer accumulation and the all-reduce
over a world of two `gloo` ranks; a rank that fails is noticed on the host (no GPU involved)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from inpc_b200.batch import BatchBuffers, accumulate_view, allreduce_buffers, partition_views


def test_partition_covers_every_view_once():
    for n_views, world in [(64, 1), (64, 2), (64, 8), (7, 4), (3, 8), (0, 2)]:
        shards = [partition_views(n_views, r, world) for r in range(world)]
        flat = sorted(i for s in shards for i in s)
        assert flat == list(range(n_views))
        assert max(map(len, shards)) - min(map(len, shards)) <= 1
    with pytest.raises(ValueError):
        partition_views(4, 2, 2)


def _view_contribution(view_index, n_leaves, n_points, n_app):
    g = torch.Generator().manual_seed(100 + view_index)
    idx = torch.randint(-1, n_leaves, (n_points,), generator=g)            # -1 marks "no sample" slots
    bw = torch.rand(n_points, generator=g)
    gf = (torch.randn((n_points, 36), generator=g) * 1e-3).to(torch.float16)
    go = torch.randn((n_points, 1), generator=g) * 1e-3
    return idx, bw, gf, go


def _accumulate(views, n_leaves=50, n_points=96, n_app=32):
    buf = BatchBuffers(n_leaves, n_app, "cpu")
    for v in views:
        accumulate_view(buf, *_view_contribution(v, n_leaves, n_points, n_app))
    return buf


def _finished(buf):
    """(max, min) with the "no sample" marker read as 0, as the update kernel does."""
    return buf.leaf.max_sampled.clone(), buf.leaf.min_sampled.clone()


def test_accumulate_matches_explicit_reductions():
    buf = _accumulate([0, 1])
    mx, mn = torch.zeros(50), torch.full((50,), float("inf"))
    app = torch.zeros(32)
    for v in (0, 1):
        idx, bw, gf, go = _view_contribution(v, 50, 96, 32)
        for i, w in zip(idx.tolist(), bw.tolist()):
            if i >= 0:
                mx[i] = max(mx[i], w)
                mn[i] = min(mn[i], w)
        for k, g in enumerate(go.reshape(-1).tolist()):
            app[k % 32] += g
    mn[torch.isinf(mn)] = 0.0
    got_mx, got_mn = _finished(buf)
    assert torch.equal(got_mx, mx) and torch.equal(got_mn, mn)
    assert torch.allclose(buf.appearance, app, atol=1e-6)
    # ragged point count takes the index_add path
    buf2 = BatchBuffers(50, 32, "cpu")
    idx, bw, gf, go = _view_contribution(0, 50, 96, 32)
    accumulate_view(buf2, idx[:90], bw[:90], gf[:90], go[:90])
    app2 = torch.zeros(32)
    for k, g in enumerate(go.reshape(-1)[:90].tolist()):
        app2[k % 32] += g
    assert torch.allclose(buf2.appearance, app2, atol=1e-6)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_views, fail_rank, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        if rank == fail_rank:
            raise RuntimeError("injected host-side failure before the exchange step")
        buf = _accumulate(partition_views(n_views, rank, world))
        allreduce_buffers(buf)
        out[rank] = (*_finished(buf), buf.appearance.clone())
    except Exception as e:  # a failed peer surfaces as an exception, never as a hang
        out[rank] = repr(e)
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _run_world(world, n_views, fail_rank=-1):
    mgr = mp.Manager()
    out = mgr.dict()
    port = _free_port()
    procs = [mp.get_context("spawn").Process(target=_worker, args=(r, world, port, n_views, fail_rank, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(90)
        assert not p.is_alive(), "rank did not finish"
    return dict(out)


def test_two_rank_allreduce_equals_single_rank_sum():
    n_views = 5
    single = _accumulate(range(n_views))
    out = _run_world(2, n_views)
    smx, smn = _finished(single)
    for r in range(2):
        mx, mn, app = out[r]
        assert torch.equal(mx, smx) and torch.equal(mn, smn)            # MAX / MIN are exact in any order
        assert torch.allclose(app, single.appearance, atol=1e-5)


def test_failed_rank_is_reported_not_hung():
    out = _run_world(2, 4, fail_rank=1)
    assert isinstance(out[1], str) and "injected" in out[1]
    # the surviving rank ends with an error from the collective (peer gone / timeout), not a result
    assert isinstance(out[0], str)
