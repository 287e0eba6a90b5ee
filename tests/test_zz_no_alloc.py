"""The non-allocating gradient-norm entry point, driven through its exported C symbol, against the regular entry
point.  Collected last so that it also runs after every other GPU test has used the device."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from loomformer_paraplex_b200.ops import native
    native.load(required=True)
    lib = ctypes.CDLL(native.so_path())
    lib.loom_grad_norm_static.restype = ctypes.c_int
    lib.loom_grad_norm_static.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_float, ctypes.c_int,
                                          ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.loom_grad_norm.restype = ctypes.c_int
    lib.loom_grad_norm.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p, ctypes.c_int,
                                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.loom_static_strerror.restype = ctypes.c_char_p
    lib.loom_static_strerror.argtypes = [ctypes.c_int]
    return lib


def test_static_scratch_grad_norm_matches_regular_entry_point_twice():
    lib = _lib()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda").manual_seed(3)
    for call, (n, nparts, max_norm) in enumerate(((1 << 22, 592, 1.55), (256 * 1001, 37, 0.0))):
        grads = torch.randn(n, device=dev, generator=g) * (0.01 if call == 0 else 3.0)
        want, got = torch.full((4,), -1.0, device=dev), torch.full((4,), -1.0, device=dev)
        atom_a, atom_b = torch.ones(4, device=dev), torch.ones(4, device=dev)
        partial = torch.empty(nparts, device=dev)
        rc = lib.loom_grad_norm(grads.data_ptr(), n, max_norm, partial.data_ptr(), nparts, want.data_ptr(),
                                atom_a.data_ptr(), stream)
        assert rc == 0
        if call == 1:
            # the first call on a device looked the array's address up; from the second call on the driver's own count
            # of free bytes must not move (torch's counter alone would not see a raw cudaMalloc inside the library)
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info(dev)[0]
        before = torch.cuda.memory_allocated()
        rc = lib.loom_grad_norm_static(grads.data_ptr(), n, max_norm, nparts, got.data_ptr(), atom_b.data_ptr(), stream)
        assert rc == 0, lib.loom_static_strerror(rc)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        if call == 1:
            assert torch.cuda.mem_get_info(dev)[0] == free_before
        ref = grads.double().norm().item()
        assert abs(got[0].item() - ref) <= 1e-4 * ref
        assert torch.allclose(got[:3], want[:3], rtol=1e-6, atol=0.0)
        assert got[2].item() == 1.0 and torch.equal(atom_a, atom_b) and atom_b[:3].abs().sum().item() == 0.0
        if max_norm > 0:
            assert abs(got[1].item() - min(1.0, max_norm / (ref + 1e-6))) < 1e-5
        else:
            assert got[1].item() == 1.0
    # a non-finite gradient raises the flag on the same shared scratch
    grads[5] = float("inf")
    rc = lib.loom_grad_norm_static(grads.data_ptr(), n, 1.0, nparts, got.data_ptr(), None, stream)
    torch.cuda.synchronize()
    assert rc == 0 and got[2].item() == 0.0 and got[1].item() == 1.0


def test_static_scratch_has_its_own_array_on_a_second_device():
    """Each device that loads the library holds its own copy of the array and its own cached address."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    lib = _lib()
    for idx in (1, 0, 1):
        dev = torch.device("cuda", idx)
        with torch.cuda.device(dev):
            stream = torch.cuda.current_stream(dev).cuda_stream
            grads = torch.full((256 * 64,), 0.5, device=dev)
            got = torch.zeros(4, device=dev)
            rc = lib.loom_grad_norm_static(grads.data_ptr(), grads.numel(), 0.0, 16, got.data_ptr(), None, stream)
            assert rc == 0, lib.loom_static_strerror(rc)
            torch.cuda.synchronize(dev)
            assert abs(got[0].item() - 0.5 * (256 * 64) ** 0.5) < 1e-3 and got[2].item() == 1.0


def test_static_scratch_refuses_what_does_not_fit():
    lib = _lib()
    dev = torch.device("cuda:0")
    grads = torch.zeros(1024, device=dev)
    stats = torch.zeros(4, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.loom_grad_norm_static(grads.data_ptr(), 1024, 1.0, 1025, stats.data_ptr(), None, stream)
    assert rc == -101 and b"1024" in lib.loom_static_strerror(rc)
    assert lib.loom_grad_norm_static(grads.data_ptr(), 1024, 1.0, 0, stats.data_ptr(), None, stream) == -101
    assert lib.loom_grad_norm_static(grads.data_ptr(), 1022, 1.0, 8, stats.data_ptr(), None, stream) == -102
    assert lib.loom_grad_norm_static(grads.data_ptr() + 4, 1020, 1.0, 8, stats.data_ptr(), None, stream) == -102
    assert lib.loom_grad_norm_static(None, 1024, 1.0, 8, stats.data_ptr(), None, stream) == -103
    torch.cuda.synchronize()
