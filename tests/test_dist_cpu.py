"""Batch sharding + the single dW all-reduce, as world-size-2 gloo ranks on CPU.
The per-rank operators are stood in for by the CPU oracle (test infrastructure): what is
under test is the sharding arithmetic, the flat-buffer reducer and the failure behaviour."""
import os
import socket
import sys
import traceback
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG, ROOT


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, scenario, q):
    try:
        for p in (ROOT, PKG):
            if p not in sys.path:
                sys.path.insert(0, p)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        import oracle
        from dwconv_b200.dist import FilterGradReducer, shard_batch, shard_bounds
        dist.init_process_group("gloo", rank=rank, world_size=world,
                                timeout=timedelta(seconds=5 if scenario == "rank_fails" else 60))
        g = torch.Generator().manual_seed(0)
        layers = [(6, 14, 3, 1, 1), (4, 9, 5, 2, 2)]  # C, H, k, s, p
        N = 7  # not divisible by the world size: ragged shards
        xs, dys, ws = [], [], []
        for C, H, k, s, p in layers:
            x = torch.randn(N, C, H, H, generator=g)
            w = torch.randn(C, 1, k, k, generator=g)
            ho = oracle.conv_out(H, k, s, p)
            dys.append(torch.randn(N, C, ho, ho, generator=g))
            xs.append(x)
            ws.append(w)
        if scenario == "rank_fails" and rank == 1:
            raise RuntimeError("injected failure before the collective")
        lo, hi = shard_bounds(N, world, rank)
        local, full_y = [], []
        for (C, H, k, s, p), x, w, dy in zip(layers, xs, ws, dys):
            xl, dyl = shard_batch(x, world, rank), shard_batch(dy, world, rank)
            assert xl.shape[0] == hi - lo
            local.append(oracle.backward_filter(xl, dyl, (k, k), s, p).float())
            # forward / backward-input need no exchange: the shard equals the slice of the whole
            y_full = oracle.forward_seq(x, w, s, p)
            assert torch.equal(oracle.forward_seq(xl, w, s, p), y_full[lo:hi])
            dx_full = oracle.backward_input_seq(dy, w, (H, H), s, p)
            assert torch.equal(oracle.backward_input_seq(dyl, w, (H, H), s, p), dx_full[lo:hi])
        red = FilterGradReducer([t.shape for t in local], "cpu")
        assert red.nbytes == 4 * sum(t.numel() for t in local)
        summed = red.reduce(local)
        for (C, H, k, s, p), x, dy, got in zip(layers, xs, dys, summed):
            truth = oracle.backward_filter(x, dy, (k, k), s, p)
            err = (got.double() - truth).abs().max().item()
            assert err <= 1e-4 * truth.abs().max().item(), err
        # a second step reuses the buffer
        again = red.reduce(local)
        assert all(torch.equal(a, b) for a, b in zip(again, summed))
        # fp16 gradients travel as fp32 and come back as fp16
        half = red.reduce([t.half() for t in local])
        assert all(h.dtype == torch.float16 for h in half)
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, f"{type(e).__name__}: {e}\n{traceback.format_exc()[-600:]}"))


def _run(scenario, world=2):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, scenario, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
    return out


def test_shard_bounds_cover_batch_exactly():
    from dwconv_b200.dist import shard_bounds
    for n in (1, 7, 8, 64, 128, 129):
        for world in (1, 2, 4, 8):
            spans = [shard_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert max(h - l for l, h in spans) - min(h - l for l, h in spans) <= 1
    with pytest.raises(ValueError):
        shard_bounds(8, 2, 2)


def test_two_rank_sharded_step_matches_single_process():
    out = _run("ok")
    assert out == {0: "ok", 1: "ok"}, out


def test_rank_failure_surfaces_as_error_not_hang():
    """Rank 1 raises before the collective; rank 0's all-reduce must end with an error
    within the process-group timeout instead of waiting forever."""
    out = _run("rank_fails")
    assert "injected failure" in out[1]
    assert out[0] != "ok"


def test_cpulist_parsing_and_binding_never_raises(tmp_path):
    from dwconv_b200.dist import _parse_cpulist, bind_to_gpu_numa_node
    assert _parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert _parse_cpulist("") == set()
    info = bind_to_gpu_numa_node(0, sysfs=str(tmp_path))  # no GPU / no sysfs here: reports, no raise
    assert info["bound"] is False
