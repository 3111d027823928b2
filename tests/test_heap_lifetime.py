"""A tensor built on symmetric-heap memory may outlive its communicator.

`heap_tensor` takes a reference on the communicator's heap; destroying the communicator while such tensors
exist stops it serving calls at once, but the heap stays mapped until the last tensor is gone, so neither the
tensor's memory nor its deleter ever dangles.  One rank on one GPU is enough to exercise the bookkeeping."""
import gc

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_heap_tensor_survives_its_communicator(native_lib):
    import flagcx_b200
    from flagcx_b200.wrapper import FLAGCXError, FLAGCXLibrary
    nat = flagcx_b200.native()
    lib = FLAGCXLibrary(native_lib)
    torch.zeros(1, device="cuda")
    comm = lib.flagcxCommInitRank(1, lib.flagcxGetUniqueId(), 0)
    a = nat.heap_tensor(comm.value, [1 << 20], torch.float32)
    b = nat.heap_tensor(comm.value, [4096], torch.bfloat16)
    a.fill_(3.0)
    b.fill_(2.0)
    torch.cuda.synchronize()
    lib.flagcxCommDestroy(comm)  # two tensors still hold heap memory
    # the handle is dead for the API ...
    with pytest.raises(FLAGCXError):
        lib.flagcxCommCount(comm)
    with pytest.raises(RuntimeError):
        nat.heap_tensor(comm.value, [16], torch.float32)
    # ... but the memory is not: kernels may still read and write it
    a.mul_(2.0)
    torch.cuda.synchronize()
    assert float(a.sum().item()) == 6.0 * (1 << 20)
    assert float(b.float().sum().item()) == 2.0 * 4096
    del a
    gc.collect()
    b.add_(1.0)
    torch.cuda.synchronize()
    assert float(b.float().max().item()) == 3.0
    del b  # the last holder: the heap is unmapped now
    gc.collect()
    torch.cuda.synchronize()
    # the device is fine and a new communicator can be made
    comm2 = lib.flagcxCommInitRank(1, lib.flagcxGetUniqueId(), 0)
    c = nat.heap_tensor(comm2.value, [1024], torch.float32)
    c.fill_(1.0)
    assert float(c.sum().item()) == 1024.0
    del c
    lib.flagcxCommDestroy(comm2)
