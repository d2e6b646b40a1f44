"""One-shot all-reduce over peer-mapped buffers (`dsv3_allreduce_oneshot`, replaces dist.all_reduce of
model.py:263-264, 691-692 for decode-sized tensors).

On one GPU two ranks are played inside one process by ONE cooperative launch (the ranks' CTAs wait for each other's
signals, so they must not be separate kernels that might never run at the same time).  Checked: the sum equals the
fp32 sum of the partials rounded to bf16, bit for bit and identically on both ranks; sequence numbers and slot
alternation over many calls of different sizes; replay inside a CUDA graph; sizes with a tail; refusal of oversized
tensors; and the bounded wait: a rank whose peer never signals returns, leaves its output untouched and reports
DSV3_ERR_DEVICE_TIMEOUT through the status words (the wait simply runs out; nothing faults, traps or hangs).
With two GPUs, two processes do the same through CUDA IPC and compare with the same reference.
"""
import ctypes
import os
import sys

import numpy as np
import pytest
import torch

from gpu_util import bf16_bits

pytestmark = pytest.mark.gpu


class Pair:
    """Ranks 0 and 1 of a world of 2 on the current GPU, wired to each other inside this process."""

    def __init__(self, max_bytes):
        from dsv3_b200 import _lib
        self._lib, self.lib = _lib, _lib.lib
        self.comms = []
        for r in range(2):
            comm = ctypes.c_void_p()
            handle = ctypes.create_string_buffer(self.lib.dsv3_p2p_handle_bytes())
            _lib.check(self.lib.dsv3_p2p_create(r, 2, max_bytes, ctypes.byref(comm), handle))
            self.comms.append(comm)
        bases = (ctypes.c_void_p * 2)(*[self.lib.dsv3_p2p_base(c) for c in self.comms])
        for c in self.comms:
            _lib.check(self.lib.dsv3_p2p_connect_local(c, bases))

    def all_reduce(self, a, b, out_a, out_b, limit_ns=0):
        st = torch.cuda.current_stream().cuda_stream
        self._lib.check(self.lib.dsv3_allreduce_oneshot_pair_on_one_gpu(
            self.comms[0], self.comms[1], a.data_ptr(), b.data_ptr(), out_a.data_ptr(), out_b.data_ptr(), a.numel(), limit_ns, st))

    def close(self):
        torch.cuda.synchronize()
        for c in self.comms:
            self.lib.dsv3_p2p_destroy(c)


def _partials(n, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(n, generator=g, device="cuda").bfloat16(), torch.randn(n, generator=g, device="cuda").bfloat16())


def _want(a, b):
    return (a.float() + b.float()).to(torch.bfloat16)


def test_two_ranks_in_one_launch_sum_bit_exactly_over_many_calls():
    import dsv3_b200
    pair = Pair(2 << 20)
    try:
        for i, n in enumerate([7168, 8 * 7168, 64 * 7168, 7168, 1000, 8, 3, 64 * 7168, 16 * 7168 + 5, 7168]):
            a, b = _partials(n, 100 + i)
            oa, ob = torch.zeros_like(a), torch.zeros_like(b)
            pair.all_reduce(a, b, oa, ob)
            torch.cuda.synchronize()
            want = _want(a, b)
            assert np.array_equal(bf16_bits(oa), bf16_bits(want)), (i, n)
            assert np.array_equal(bf16_bits(ob), bf16_bits(want)), (i, n)
        # in place
        a, b = _partials(4 * 7168, 7)
        want = _want(a, b)
        pair.all_reduce(a, b, a, b)
        torch.cuda.synchronize()
        assert torch.equal(a, want) and torch.equal(b, want)
        dsv3_b200.check_device_status()
    finally:
        pair.close()


def test_all_reduce_replayed_in_a_cuda_graph():
    import dsv3_b200
    pair = Pair(1 << 20)
    try:
        a, b = _partials(16 * 7168, 21)
        oa, ob = torch.zeros_like(a), torch.zeros_like(b)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            pair.all_reduce(a, b, oa, ob)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                pair.all_reduce(a, b, oa, ob)         # three launches per replay: the slot parity differs between replays
                pair.all_reduce(oa, ob, oa, ob)
                pair.all_reduce(a, b, oa, ob)
            for rep in range(5):
                a.copy_(_partials(16 * 7168, 30 + rep)[0])      # new partials before every replay
                oa.zero_(); ob.zero_()
                g.replay()
                side.synchronize()
                want = _want(a, b)
                assert torch.equal(oa, want) and torch.equal(ob, want), rep
        dsv3_b200.check_device_status()
    finally:
        pair.close()


def test_all_reduce_refuses_a_tensor_larger_than_the_buffer():
    from dsv3_b200 import _lib
    pair = Pair(4096)
    try:
        a, b = _partials(4096, 1)
        with pytest.raises(_lib.Dsv3Error) as e:
            pair.all_reduce(a, b, a.clone(), b.clone())
        assert e.value.status == -4
    finally:
        pair.close()


def test_bounded_wait_runs_out_when_the_peer_never_signals():
    """Rank 0 is launched alone: its peer's flag is never set.  The wait gives up after its limit (2 ms here), the
    kernel returns normally, the output keeps its old contents and the status words say which wait ran out."""
    import dsv3_b200
    from dsv3_b200 import _lib
    lib = _lib.lib
    pair = Pair(1 << 20)
    try:
        a, _ = _partials(7168, 3)
        out = torch.full_like(a, 5.0)
        _lib.check(lib.dsv3_allreduce_oneshot(pair.comms[0], a.data_ptr(), out.data_ptr(), a.numel(), 2_000_000,
                                              torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()                                  # returns: nothing hangs
        assert bool((out == 5.0).all())
        detail = (ctypes.c_uint32 * 4)()
        rc = lib.dsv3_check_device_status(torch.cuda.current_stream().cuda_stream, detail)
        assert rc == _lib.ERR_DEVICE_TIMEOUT
        assert detail[1] == 10 and (detail[3] >> 16) == 0 and (detail[3] & 0xFFFF) == 1     # rank 0 waited for peer 1
        dsv3_b200.check_device_status()                           # cleared by the read above
    finally:
        pair.close()


def _two_gpu_worker(rank, world, port, ok_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    import dsv3_b200
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ar = dsv3_b200.P2PAllReduce(max_bytes=1 << 20)
    try:
        for i, n in enumerate([7168, 64 * 7168, 1000, 7168 * 3 + 2]):
            g = torch.Generator(device="cuda").manual_seed(500 + i)           # same stream on both ranks
            parts = [torch.randn(n, generator=g, device="cuda").bfloat16() for _ in range(world)]
            mine = parts[rank].clone()
            ar.all_reduce(mine)
            want = sum(p.float() for p in parts).to(torch.bfloat16)
            torch.cuda.synchronize()
            assert torch.equal(mine, want), (rank, i)
            ref = parts[rank].clone()
            dist.all_reduce(ref)                                             # NCCL: same sum up to its own rounding order
            assert (ref.float() - mine.float()).abs().max().item() <= 0.0625 * want.float().abs().max().item()
        dsv3_b200.check_device_status()
        open(ok_path + f".{rank}", "w").write("ok")
    finally:
        ar.close()
        dist.destroy_process_group()


def test_two_processes_on_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ok = str(tmp_path / "ok")
    mp.spawn(_two_gpu_worker, args=(2, 29533, ok), nprocs=2, join=True)
    assert os.path.exists(ok + ".0") and os.path.exists(ok + ".1")
