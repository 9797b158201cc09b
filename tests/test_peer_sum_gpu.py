"""The loss-sum exchange over peer memory (tb200_loss_sum_exchange; no counterpart in the
single-GPU reference).  On one GPU: a world of one, and the time limit of the wait (a peer that
never writes -- nothing is made to hang or fault: the wait is bounded and the kernel returns).
With two or more GPUs: two ranks as child processes, one per GPU, against an NCCL-free sum."""
import ctypes
import os
import subprocess
import sys

import pytest
import torch

import abi
from transducer_b200.errors import DeviceStatusError

pytestmark = pytest.mark.gpu
lib = abi.lib


def alloc():
    p = ctypes.c_void_p()
    abi.check(lib.tb200_peer_alloc(ctypes.byref(p)))
    return p


def test_world_of_one_returns_its_own_sum():
    mine = alloc()
    try:
        ptrs = (ctypes.c_void_p * 1)(mine.value)
        total = torch.zeros(1, device="cuda")
        abi.use_torch_stream()
        for seq, x in enumerate((3.25, -7.5, 1e-3), start=1):
            loss = torch.full((1,), x, device="cuda")
            abi.check(lib.tb200_loss_sum_exchange(abi.ptr(loss), ptrs, 0, 1, seq, abi.ptr(total), 0))
            torch.cuda.synchronize()
            assert float(total) == float(loss)
        abi.check(lib.tb200_check_status())
    finally:
        lib.tb200_peer_free(mine)


def test_a_silent_peer_runs_into_the_time_limit_and_is_reported():
    mine, other = alloc(), alloc()   # `other` stands for a peer that never takes part
    try:
        ptrs = (ctypes.c_void_p * 2)(mine.value, other.value)
        total = torch.zeros(1, device="cuda")
        loss = torch.ones(1, device="cuda")
        abi.use_torch_stream()
        abi.check(lib.tb200_loss_sum_exchange(abi.ptr(loss), ptrs, 0, 2, 1, abi.ptr(total), 2000))
        torch.cuda.synchronize()
        assert torch.isnan(total).all()
        with pytest.raises(DeviceStatusError) as err:
            abi.check(lib.tb200_check_status())
        assert "peer" in str(err.value)
        abi.check(lib.tb200_check_status())   # the word was cleared; the context still works
        assert float((loss + 1).sum()) == 2.0
    finally:
        lib.tb200_peer_free(mine)
        lib.tb200_peer_free(other)


def test_bad_arguments():
    total = torch.zeros(1, device="cuda")
    loss = torch.ones(1, device="cuda")
    ptrs = (ctypes.c_void_p * 1)(0)
    with pytest.raises(ValueError):
        abi.check(lib.tb200_loss_sum_exchange(abi.ptr(loss), ptrs, 0, 1, 1, abi.ptr(total), 0))
    with pytest.raises(ValueError):
        abi.check(lib.tb200_loss_sum_exchange(abi.ptr(loss), ptrs, 0, 33, 1, abi.ptr(total), 0))


CHILD = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["TB200_REPO"])
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("gloo")
from transducer_b200.distributed import PeerLossSum
from transducer_b200.torch_binding import check_device_status
red = PeerLossSum()
for step in range(200):
    mine = torch.full((1,), (rank + 1) * 0.5 + step, device="cuda")
    total = red(mine)
    want = sum((r + 1) * 0.5 + step for r in range(world))
    if step % 50 == 0:
        torch.cuda.synchronize()
        assert float(total) == want, (rank, step, float(total), want)
torch.cuda.synchronize()
assert float(total) == want
check_device_status()
red.close()
dist.destroy_process_group()
print("rank %d ok" % rank)
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_on_two_gpus():
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29731", WORLD_SIZE="2",
               TB200_REPO=repo, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, "-c", CHILD], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(2)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=180)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "rank %d ok" % r in out, out[-2000:]
