"""Failure detection without a GPU fault.

On the GPU every wait is bounded: a barrier whose peer never signals returns after its limit and leaves
CGX_ETIMEDOUT in the device status word; the context stays usable.  The test makes the wait run out by pointing the
"peer" flag array at local memory nobody writes.  Nothing traps, faults or spins for ever.

On the host a rank that dies before the exchange must not leave the others hanging: the size-table all-gather of
the surviving rank ends with an error inside the process group's timeout (gloo ranks on CPU)."""
import ctypes as C
import os
import socket
import sys
import time
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.gpu
def test_peer_barrier_wait_runs_out_and_reports(cuda_device):
    from diff_gaussian_rasterization import _lib

    l = _lib.lib()
    dev = cuda_device
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = C.c_int(-1)
    assert l.cgx_device_status(C.byref(status), st) == 0 and status.value == 0
    mine = torch.zeros(64, dtype=torch.int32, device=dev)       # this rank's flag words
    silent = torch.zeros(64, dtype=torch.int32, device=dev)     # stands for a peer that never signals
    ptrs = (C.c_void_p * 2)(mine.data_ptr(), silent.data_ptr())
    limit = 4_000_000                                            # about 2 ms of SM clocks
    t0 = time.perf_counter()
    assert l.cgx_peer_barrier_limited(2, 0, ptrs, 1, limit, st) == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0                        # returned: did not wait for the default 2 s bound
    # the asynchronous read (pinned memory, no clearing) and the synchronous one agree
    pinned = torch.zeros(4, dtype=torch.int32).pin_memory()
    assert l.cgx_device_status_async(C.c_void_p(pinned.data_ptr()), st) == 0
    torch.cuda.synchronize()
    assert pinned.tolist() == [0, _lib.CGX_ETIMEDOUT, 0, 0]
    assert l.cgx_device_status(C.byref(status), st) == 0 and status.value == _lib.CGX_ETIMEDOUT
    assert l.cgx_device_status(C.byref(status), st) == 0 and status.value == 0      # read clears
    assert int(mine[0]) == 1 and int(silent[0]) == 1 and int(mine[1]) == 0          # signalled, never answered
    # the same barrier with a peer that has already signalled passes, and the context is still good
    mine[1] = 2
    assert l.cgx_peer_barrier_limited(2, 0, ptrs, 2, limit, st) == 0
    torch.cuda.synchronize()
    assert l.cgx_device_status(C.byref(status), st) == 0 and status.value == 0
    assert l.cgx_peer_barrier_limited(2, 5, ptrs, 3, limit, st) == _lib.CGX_EINVAL    # rank outside the group


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_dies_worker(rank, ws, port, out_dir):
    for p in (ROOT, ROOT / "citygs-x_b200", ROOT / "tests"):
        sys.path.insert(0, str(p))
    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=ws, timeout=datetime.timedelta(seconds=8))
    from cgx import exchange

    dist.barrier()
    if rank == 1:
        os._exit(17)                 # dies between steps, with nothing in flight
    table = torch.zeros(4, dtype=torch.int32)
    t0 = time.perf_counter()
    try:
        exchange._gather_table(table, 4, None, None, ws)
        outcome = "returned"
    except Exception as e:          # the collective ends with an error instead of hanging
        outcome = "raised:" + type(e).__name__
    with open(os.path.join(out_dir, "rank0.txt"), "w") as f:
        f.write(f"{outcome} {time.perf_counter() - t0:.2f}")
    os._exit(0)


def test_surviving_rank_gets_an_error_when_its_peer_dies(tmp_path):
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_rank_dies_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=90)
    assert all(not p.is_alive() for p in procs), "a rank is still waiting for its dead peer"
    assert procs[1].exitcode == 17
    outcome, seconds = (tmp_path / "rank0.txt").read_text().split()
    assert outcome.startswith("raised:"), outcome
    assert float(seconds) < 60.0


@pytest.mark.gpu
def test_small_read_back_by_kernel(cuda_device):
    """cgx_post_words: device words arrive in page-locked host memory once the stream has been waited for; pageable
    memory and misaligned pointers are refused without a launch."""
    from diff_gaussian_rasterization import _lib

    l = _lib.lib()
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    src = torch.arange(1000, dtype=torch.int32, device=cuda_device) * 7 - 3
    dst = torch.zeros(1000, dtype=torch.int32).pin_memory()
    assert l.cgx_post_words(C.c_void_p(src.data_ptr()), C.c_void_p(dst.data_ptr()), 1000, st) == 0
    torch.cuda.synchronize()
    assert torch.equal(dst, src.cpu())
    assert l.cgx_post_words(C.c_void_p(src.data_ptr()), C.c_void_p(dst.data_ptr()), 0, st) == 0
    pageable = torch.zeros(16, dtype=torch.int32)
    assert l.cgx_post_words(C.c_void_p(src.data_ptr()), C.c_void_p(pageable.data_ptr()), 16, st) == _lib.CGX_EINVAL
    assert l.cgx_post_words(C.c_void_p(src.data_ptr() + 2), C.c_void_p(dst.data_ptr()), 4, st) == _lib.CGX_EINVAL
    torch.cuda.synchronize()
    status = C.c_int(-1)
    assert l.cgx_device_status(C.byref(status), st) == 0 and status.value == 0
