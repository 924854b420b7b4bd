"""Two GPUs, one process each: the one-launch peer all-reduce + norm (``fl_allreduce_rmsnorm``)
against ``step_ops.rmsnorm`` of the summed rows, eagerly and replayed from a CUDA graph, and its
bounded wait: a rank that publishes nothing makes the call give up with status 1, the GPUs keep
answering and the next call is right again.  Skipped where fewer than two GPUs are visible.

The ranks talk through a ``gloo`` group on the host (handle exchange only): no NCCL, no NVLS
object, plain peer stores."""

from __future__ import annotations

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu
WIDTH, ROWS_MAX = 2048, 16


def _inputs(call: int, rows: int, world: int):
    """The same tensors on every rank: the partial rows of all ranks, an addend, a residual."""

    g = torch.Generator().manual_seed(1000 + call)
    parts = [(torch.randn(rows, 1, WIDTH, generator=g) * 2).to(torch.bfloat16) for _ in range(world)]
    addend = torch.randn(rows, 1, WIDTH, generator=g).to(torch.bfloat16)
    residual = torch.randn(rows, 1, WIDTH, generator=g).to(torch.bfloat16)
    return parts, addend, residual


def _worker(rank: int, world: int, port: int, results) -> None:
    import torch.distributed as dist

    from flashloop_b200 import step_ops
    from flashloop_b200.tensor_parallel import PeerAllReduce

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    out = {}
    try:
        comm = PeerAllReduce(dist.group.WORLD, rows_max=ROWS_MAX, width=WIDTH, device=torch.device("cuda", rank),
                             wait_limit=400_000)
        g = torch.Generator().manual_seed(5)
        w1 = (1 + 0.1 * torch.randn(WIDTH, generator=g)).to(torch.bfloat16).cuda()
        w2 = (1 + 0.1 * torch.randn(WIDTH, generator=g)).to(torch.bfloat16).cuda()

        def expected(call, rows, variant):
            parts, addend, residual = _inputs(call, rows, world)
            total = parts[0].cuda()
            for p in parts[1:]:
                total = total + p.cuda()  # two ranks: one bfloat16 rounding of the float32 sum
            if variant == "sum":
                return total, None, total
            if variant == "addend":
                total = addend.cuda() + total
            hidden, x = step_ops.rmsnorm(total, w1, 1e-6, residual=residual.cuda(), weight2=w2, eps2=1e-5)
            return hidden, x, total

        def run(call, rows, variant, **kw):
            parts, addend, residual = _inputs(call, rows, world)
            mine = parts[rank].cuda()
            if variant == "sum":
                return comm.reduce_norm(mine, **kw)
            return comm.reduce_norm(mine, w1, 1e-6, residual=residual.cuda(), weight2=w2, eps2=1e-5,
                                    addend=addend.cuda() if variant == "addend" else None, want_sum=True, **kw)

        # ---- eager calls: both slot halves, ragged row counts, all variants
        exact = True
        for call in range(24):
            rows = (1, 16, 5, 3)[call % 4]
            variant = ("sum", "norm", "addend")[call % 3]
            got = run(call, rows, variant)
            want = expected(call, rows, variant)
            for a, b in zip(got, want):
                exact &= (a is None and b is None) or bool(torch.equal(a, b))
        out["eager_exact"] = exact
        out["status_after_eager"] = comm.status()

        # ---- a recorded step of six calls, replayed
        dist.barrier()
        parts, addend, residual = _inputs(99, 8, world)
        static_in = parts[rank].cuda()
        static_res, static_add = residual.cuda(), addend.cuda()
        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph):
            hidden = static_res
            for _ in range(3):
                hidden, x, _ = comm.reduce_norm(static_in, w1, 1e-6, residual=hidden, weight2=w2, eps2=1e-5)
                hidden, x, _ = comm.reduce_norm(x, w1, 1e-6, residual=hidden, weight2=w2, eps2=1e-5,
                                                addend=static_add)
        total = parts[0].cuda() + parts[1].cuda()
        want_h = static_res
        for _ in range(3):
            want_h, want_x = step_ops.rmsnorm(total, w1, 1e-6, residual=want_h, weight2=w2, eps2=1e-5)
            # every rank feeds the same x: the sum is world * x, one rounding
            doubled = static_add + (want_x + want_x)
            want_h, want_x = step_ops.rmsnorm(doubled, w1, 1e-6, residual=want_h, weight2=w2, eps2=1e-5)
        replays = True
        for _ in range(5):
            graph.replay()
            torch.cuda.synchronize()
            replays &= bool(torch.equal(hidden, want_h)) and bool(torch.equal(x, want_x))
        out["graph_exact"] = replays
        out["status_after_graph"] = comm.status()

        # ---- the bounded wait: rank 1 publishes nothing in one call
        dist.barrier()
        torch.cuda.synchronize()
        run(200, 4, "norm", _skip_store=(rank == 1))
        out["status_after_skip"] = comm.status(reset=True)
        dist.barrier()
        out["status_after_reset"] = comm.status()
        got = run(201, 4, "addend")
        want = expected(201, 4, "addend")
        out["recovered"] = all(bool(torch.equal(a, b)) for a, b in zip(got, want))
        out["status_at_end"] = comm.status()
        torch.cuda.synchronize()
        dist.barrier()
        comm.close()
        results[rank] = out
    finally:
        dist.destroy_process_group()


def test_peer_allreduce_two_ranks():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(150)
    stuck = [p for p in procs if p.exitcode is None]
    for p in stuck:
        p.terminate()
    assert not stuck and all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    for rank in range(2):
        r = results[rank]
        assert r["eager_exact"] and r["status_after_eager"] == 0, r
        assert r["graph_exact"] and r["status_after_graph"] == 0, r
        assert r["status_after_skip"] == 1, r        # the wait for rank 1's rows ran out on both ranks
        assert r["status_after_reset"] == 0 and r["recovered"] and r["status_at_end"] == 0, r


def test_communicator_rejects_bad_shapes():
    import ctypes

    from flashloop_b200 import _native

    lib = _native.load()
    comm, handle = ctypes.c_void_p(), ctypes.create_string_buffer(int(lib.fl_comm_handle_bytes()))
    assert lib.fl_comm_create(0, 9, 4, 256, ctypes.byref(comm), handle) != 0       # more than 8 ranks
    assert lib.fl_comm_create(0, 2, 4, 100, ctypes.byref(comm), handle) != 0       # width not a multiple of 8
    assert lib.fl_comm_create(0, 2, 4, 16384, ctypes.byref(comm), handle) != 0     # wider than a CTA covers
    assert b"fl_comm_create" in lib.fl_last_error()
    # one rank: the sum is the input, the norms those of fl_rmsnorm
    from flashloop_b200 import step_ops

    assert lib.fl_comm_create(0, 1, 4, 256, ctypes.byref(comm), handle) == 0
    assert lib.fl_comm_connect(comm, handle.raw) == 0
    x = torch.randn(3, 1, 256, device="cuda").to(torch.bfloat16)
    w = torch.ones(256, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(x)
    assert lib.fl_allreduce_rmsnorm(comm, x.data_ptr(), None, None, w.data_ptr(), 1e-6, None, 0.0, 5, None,
                                    out.data_ptr(), None, 0, 0, _native.current_stream(x.device)) != 0  # rows > max
    assert lib.fl_allreduce_rmsnorm(comm, x.data_ptr(), None, None, w.data_ptr(), 1e-6, None, 0.0, 3, None,
                                    out.data_ptr(), None, 0, 0, _native.current_stream(x.device)) == 0
    assert torch.equal(out, step_ops.rmsnorm(x, w, 1e-6))
    word = ctypes.c_int32(-1)
    assert lib.fl_comm_status(comm, ctypes.byref(word), 0, _native.current_stream(x.device)) == 0 and word.value == 0
    assert lib.fl_comm_destroy(comm) == 0
