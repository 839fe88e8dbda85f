"""Bounded device-side waits that run out: the kernel returns, the status word carries the code of the wait, the
host call that reads it raises, and the CUDA context stays usable.  The waits are made to run out with flags that
nothing ever sets (no fault, no trap, no endless loop)."""
import pytest
import torch

from vllm_kunlun_b200.ops import _ext

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_flag_wait_runs_out_and_sets_the_status_word():
    C = _ext.C()
    flags = torch.zeros(8, dtype=torch.int32, device=DEV)   # arrival counters nobody bumps
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    C.sp_wait(flags.data_ptr(), 4, 1, 1000, status)           # 4 token tiles, expect 1 arrival, 1000 polls
    torch.cuda.synchronize()
    assert int(status.item()) == 400
    # the context is alive and a satisfied wait leaves the word alone
    status.zero_()
    flags.fill_(1)
    C.sp_wait(flags.data_ptr(), 4, 1, 1000, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.ones(4, device=DEV).sum().item() == 4.0


def test_allreduce_wait_for_a_silent_peer_runs_out_and_check_status_raises():
    """Two-rank low-latency all-reduce on ONE GPU where the peer never pushes: rank 0 writes its units into the
    second rank's slots of the shared buffer and then polls its own slots, which nothing fills."""
    C = _ext.C()
    rows, H = 4, 256
    slot_bytes = rows * H * 4
    buf = torch.zeros(2 * 2 * slot_bytes, dtype=torch.uint8, device=DEV)   # [parity][source] slots
    bufs = [buf.data_ptr(), buf.data_ptr() + 0]                             # both "ranks" map the same memory
    x = torch.randn(rows, H, device=DEV).to(torch.bfloat16)
    out = torch.empty_like(x)
    epochs = torch.zeros(128, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    C.ll_allreduce(bufs, x, out, None, None, epochs, status, slot_bytes, 0, 0.0, False, rows, 2000, False)
    torch.cuda.synchronize()
    assert int(status.item()) == 211, "wait on the slots of rank 1 must give up with code 210 + rank"
    assert int(epochs[0].item()) == 1 and int(epochs[1].item()) == 0   # the call still completed and re-armed its ticket

    class P:  # the host-side reader of the word
        pass
    from vllm_kunlun_b200.parallel.symm_mem import PeerBuffers
    p = P()
    p.status = status
    with pytest.raises(RuntimeError, match="code 211"):
        PeerBuffers.check_status(p)


def test_step_handle_raises_on_a_nonzero_status_word():
    from vllm_kunlun_b200.engine.runner import DeviceWaitTimeout, StepHandle
    status = torch.tensor([0, 400], dtype=torch.int32, device=DEV)
    host = torch.zeros(2, dtype=torch.int32).pin_memory()
    host.copy_(status, non_blocking=True)
    ev = torch.cuda.Event()
    ev.record()
    h = StepHandle(None, [], [], torch.zeros(1), torch.tensor([3]), ev, status_cpu=host, status_names=("gemm", "tp_peer"))
    with pytest.raises(DeviceWaitTimeout, match="tp_peer=400"):
        h.wait()
