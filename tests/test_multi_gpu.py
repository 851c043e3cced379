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


def _worker(rank, world, port, q):
    try:
        for p in (ROOT, PKG):
            if p not in sys.path:
                sys.path.insert(0, p)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
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


def test_two_gpu_batch_sharding_matches_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 CUDA devices")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = dict(q.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert out == {0: "ok", 1: "ok"}, out
