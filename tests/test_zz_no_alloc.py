"""The allocation-free arg-max entry point, called through its exported C symbol.

Some users of this library cannot allocate device memory when they call it (a host runtime that
owns the whole device budget and passes raw pointers, or a latency-critical loop that must not
touch the driver's allocator).  For them ``b200_argmax_noalloc`` keeps its scratch in a static
device array.  This test drives it with ctypes exactly as such a caller would - pointers in,
nothing allocated by the call - and checks it against the regular entry point twice in a row
(the scratch array is shared between calls and keeps the previous call's contents)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_argmax_noalloc_matches_regular_entry_point():
    from vllm_kunlun_b200 import ops
    from vllm_kunlun_b200.ops import _ext
    assert _ext.so_path() is not None, "extension not built"
    lib = ctypes.CDLL(_ext.so_path())
    fn = lib.b200_argmax_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_int64, ctypes.c_int,
                   ctypes.c_void_p]
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream().cuda_stream
    codes = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
    # inputs and outputs are allocated up front; the calls under test allocate nothing
    cases = [(16, 128256, torch.bfloat16), (5, 1000, torch.float32), (300, 32000, torch.float16)]
    tensors = [((torch.randn(r, v, device=dev) * 3).to(dt), torch.full((r,), -7, dtype=torch.int64, device=dev))
               for r, v, dt in cases]
    torch.cuda.synchronize()
    for round_ in range(2):  # two calls in a row share the static scratch
        for (logits, out), (r, v, dt) in zip(tensors, cases):
            out.fill_(-7)
            before = torch.cuda.memory_allocated(dev)
            if round_ == 1:  # after the first call per device (which resolves the symbol) the driver must not
                torch.cuda.synchronize()  # hand out a single byte either: compare the device-wide free memory
                free_before = torch.cuda.mem_get_info(dev)[0]
            rc = fn(out.data_ptr(), logits.data_ptr(), r, v, logits.stride(0), codes[dt], stream)
            assert rc == 0, rc
            assert torch.cuda.memory_allocated(dev) == before
            torch.cuda.synchronize()
            if round_ == 1 and torch.cuda.mem_get_info(dev)[0] < free_before:
                # free memory is a device-wide figure: make sure it was this call and not a neighbour process
                free_before = torch.cuda.mem_get_info(dev)[0]
                assert fn(out.data_ptr(), logits.data_ptr(), r, v, logits.stride(0), codes[dt], stream) == 0
                torch.cuda.synchronize()
                assert torch.cuda.mem_get_info(dev)[0] >= free_before, "the call took memory from the driver"
            want = ops.argmax(logits)
            assert torch.equal(out, want), (round_, r, v, dt)
            assert torch.equal(out.cpu(), logits.float().argmax(-1).cpu())
    # sizes beyond the stated maximum are refused, and nothing is written
    big = torch.zeros(4096, 64, device=dev)
    out = torch.full((4096,), -7, dtype=torch.int64, device=dev)
    assert fn(out.data_ptr(), big.data_ptr(), 4096, 64, 64, 0, stream) == 22
    torch.cuda.synchronize()
    assert int(out.min()) == -7 and int(out.max()) == -7
    # malformed arguments: rows that would overlap, an unknown element type, nothing to do
    small = torch.zeros(4, 64, device=dev)
    out4 = torch.full((4,), -7, dtype=torch.int64, device=dev)
    assert fn(out4.data_ptr(), small.data_ptr(), 4, 64, 32, 0, stream) == 22
    assert fn(out4.data_ptr(), small.data_ptr(), 4, 64, 64, 9, stream) == 22
    assert fn(out4.data_ptr(), small.data_ptr(), 0, 64, 64, 0, stream) == 0
    torch.cuda.synchronize()
    assert int(out4.min()) == -7
