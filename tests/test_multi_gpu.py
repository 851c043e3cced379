"""Batch sharding over 2 GPUs with the real kernels and NCCL: y and dx of the shards are the
slices of the single-GPU result bit for bit; the all-reduced dW matches the fp64 oracle on the
whole batch.  Needs 2 CUDA devices; skipped otherwise."""
import os
import socket
import sys
import traceback

import pytest
import torch

from conftest import PKG, ROOT

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q, scenario="sharding"):
    try:
        for p in (ROOT, PKG):
            if p not in sys.path:
                sys.path.insert(0, p)
        # plain peer loads / stores only: no NVLink multicast objects in a test where a rank
        # may stop taking part
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        if scenario != "sharding":
            return _exchange_scenario(rank, world, q, scenario)
        import torch.distributed as dist
        import dwconv_b200
        import oracle
        from dwconv_b200.dist import FilterGradReducer, PeerFilterExchange, shard_batch, shard_bounds
        from dwconv_b200 import _lib
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world,
                                device_id=torch.device("cuda", rank))
        layers = [(12, 14, 3, 1, 1, torch.float32), (6, 28, 5, 2, 2, torch.float32),
                  (8, 28, 7, 1, 3, torch.float16)]
        N = 10
        g = torch.Generator().manual_seed(3)
        grads, checks = [], []
        for (C, H, k, s, p, dt) in layers:
            x = torch.randn(N, C, H, H, generator=g).to(dt)
            w = (torch.randn(C, 1, k, k, generator=g) / k).to(dt)
            ho = oracle.conv_out(H, k, s, p)
            dy = torch.randn(N, C, ho, ho, generator=g).to(dt)
            lo, hi = shard_bounds(N, world, rank)
            xs = shard_batch(x, world, rank).cuda().requires_grad_(True)
            ws = w.cuda().requires_grad_(True)
            y = dwconv_b200.depthwise_conv2d(xs, ws, stride=s, padding=p)
            y.backward(shard_batch(dy, world, rank).cuda())
            assert torch.equal(y.detach().cpu(), oracle.forward_seq(x, w, s, p)[lo:hi])
            assert torch.equal(xs.grad.cpu(), oracle.backward_input_seq(dy, w, (H, H), s, p)[lo:hi])
            grads.append(ws.grad)
            checks.append((x, dy, k, s, p, dt))
            # the same sum made inside the filter-gradient kernel by peer stores: three calls
            # in a row (both halves of the exchange buffer get reused), identical on both ranks
            ex = PeerFilterExchange(C, k, dt, torch.device("cuda", rank))
            truth = oracle.backward_filter(x, dy, (k, k), s, p)
            rel = 1e-2 if dt == torch.float16 else 1e-4
            for _ in range(3):
                got = ex.backward_filter(xs.detach(), shard_batch(dy, world, rank).cuda(), s, p)
                both = [torch.empty_like(got) for _ in range(world)]
                dist.all_gather(both, got)
                assert torch.equal(both[0], both[1]), "ranks disagree on the exchanged dW"
                err = (got.double().cpu() - truth).abs().max().item()
                assert err <= rel * truth.abs().max().item(), err
            # the whole sum inside the finishing kernel (it waits for the peer's values itself),
            # interleaved with the pipelined form on the same object
            dys0 = shard_batch(dy, world, rank).cuda()
            for rep in range(3):
                got2 = ex.allreduce_backward_filter(xs.detach(), dys0, s, p)
                torch.cuda.synchronize()
                assert torch.equal(got2, got), "all-reduce form differs from start + finish"
                if rep == 1:
                    assert torch.equal(ex.backward_filter(xs.detach(), dys0, s, p), got)
            # pipelined form: the second start() delivers the first call's sum
            dys = shard_batch(dy, world, rank).cuda()
            first = torch.full_like(got, float("nan"))
            ex.start(xs.detach(), dys, s, p)
            ex.start(xs.detach() * 2, dys, s, p, dw_prev=first)
            second = ex.finish()
            torch.cuda.synchronize()
            assert torch.equal(first, got)
            err = (second.double().cpu() - 2 * truth).abs().max().item()
            assert err <= 2 * rel * truth.abs().max().item(), err
            assert _lib.lib.dwconv_b200_device_status() == 0
            ex.close()
        red = FilterGradReducer([t.shape for t in grads], torch.device("cuda", rank))
        summed = red.reduce(grads)
        torch.cuda.synchronize()
        for got, (x, dy, k, s, p, dt) in zip(summed, checks):
            truth = oracle.backward_filter(x, dy, (k, k), s, p)
            rel = 1e-2 if dt == torch.float16 else 1e-4
            err = (got.double().cpu() - truth).abs().max().item()
            assert err <= rel * truth.abs().max().item(), err
            assert got.dtype == dt
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, f"{type(e).__name__}: {e}\n{traceback.format_exc()[-800:]}"))


def _exchange_scenario(rank, world, q, scenario):
    """Two more uses of the in-kernel exchange on real GPUs.

    "uneven":   six pipelined calls queued back to back while rank 1's host falls behind
                (it sleeps between calls): every call must still deliver the sum of the call
                before it, identical on both ranks, with no wait expiring.
    "skipped":  rank 1 leaves out one call.  Rank 0's wait for the missing words is bounded:
                after about two seconds its kernel gives up, the call returns, bit 2 of
                dwconv_b200_device_status is set and the context stays usable.
    """
    import time
    import torch.distributed as dist
    import oracle
    from dwconv_b200 import _lib
    from dwconv_b200.dist import PeerFilterExchange, shard_batch
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    C, H, k, s, p, dt, N = 12, 14, 3, 1, 1, torch.float32, 8
    g = torch.Generator().manual_seed(5)
    ncalls = 6
    xs, dys, truth = [], [], []
    for i in range(ncalls):
        x = torch.randn(N, C, H, H, generator=g)
        dy = torch.randn(N, C, H, H, generator=g)
        truth.append(oracle.backward_filter(x, dy, (k, k), s, p))
        xs.append(shard_batch(x, world, rank).contiguous().to(dev))
        dys.append(shard_batch(dy, world, rank).contiguous().to(dev))
    ex = PeerFilterExchange(C, k, dt, dev)
    if scenario == "uneven":
        for rep in range(3):
            prev = [torch.full((C, 1, k, k), float("nan"), device=dev) for _ in range(ncalls)]
            torch.cuda.synchronize()
            dist.barrier()
            for i in range(ncalls):
                if rank == 1 and i % 2 == 1:
                    time.sleep(0.05)
                ex.start(xs[i], dys[i], s, p, dw_prev=prev[i])
            last = ex.finish()
            torch.cuda.synchronize()
            got = prev[1:] + [last]
            for i, t in enumerate(got):
                err = (t.double().cpu() - truth[i]).abs().max().item()
                assert err <= 1e-4 * truth[i].abs().max().item(), (rep, i, err)
                both = [torch.empty_like(t) for _ in range(world)]
                dist.all_gather(both, t)
                assert all(torch.equal(both[0], b) for b in both[1:]), "ranks disagree"
            assert _lib.lib.dwconv_b200_device_status() == 0
    else:
        got = ex.backward_filter(xs[0], dys[0], s, p)
        assert _lib.lib.dwconv_b200_device_status() == 0
        err = (got.double().cpu() - truth[0]).abs().max().item()
        assert err <= 1e-4 * truth[0].abs().max().item()
        dist.barrier()
        if rank == 0:
            t0 = time.perf_counter()
            ex.start(xs[1], dys[1], s, p)   # rank 1 never makes this call
            ex.finish()                     # so its words never arrive
            status = _lib.lib.dwconv_b200_device_status()   # synchronises
            waited = time.perf_counter() - t0
            assert status == 4, f"expected the exchange flag alone, got {status}"
            assert 1.0 < waited < 30.0, waited
            # the context is still usable: a plain call works and raises nothing
            dw = torch.empty((C, 1, k, k), device=dev)
            y = torch.empty_like(dys[0])
            shape = _lib.Shape(xs[0].shape[0], C, H, H, k, k, s, s, p, p, H, H)
            w = torch.randn(C, 1, k, k, device=dev)
            _lib.check(_lib.lib.dwconv_b200_forward(xs[0].data_ptr(), w.data_ptr(), y.data_ptr(),
                                                    _lib.F32, shape, None), "forward")
            assert _lib.lib.dwconv_b200_device_status() == 0
    torch.cuda.synchronize()
    ex.close()   # collective: barrier inside
    dist.destroy_process_group()
    q.put((rank, "ok"))


def _run_two_ranks(scenario, timeout=300):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 CUDA devices")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, scenario)) for r in range(2)]
    for p in procs:
        p.start()
    out = dict(q.get(timeout=timeout) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert out == {0: "ok", 1: "ok"}, out


def test_two_gpu_batch_sharding_matches_single_gpu():
    _run_two_ranks("sharding")


def test_two_gpu_exchange_with_one_rank_falling_behind():
    _run_two_ranks("uneven")


def test_two_gpu_exchange_wait_is_bounded_when_a_rank_skips_a_call():
    _run_two_ranks("skipped")
