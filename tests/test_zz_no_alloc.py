"""The allocation-free GEMV entry point against the regular one, through the C ABI (needs a B200).

Collected last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def test_static_scratch_gemv_matches_the_workspace_gemv_twice_in_a_row(orc):
    """A caller that may not allocate device memory passes inputs and outputs only; the partial sums live in
    the library's own fixed array.  Both calls must reproduce grb_bxr_gemv bit for bit, the second one starting
    from whatever the first left in the shared array."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from georefine_b200 import _native
    from georefine_b200.resident import ResidentWeight

    lib = _native.lib()
    dev = torch.device("cuda:0")
    words = orc.synthetic_weight_words(1024, 4096, 41)      # 8 row blocks shared by 148 workers: many partial tiles
    r = ResidentWeight.from_words(words, dev, layout="rans")   # the layout the CUDA-core GEMV decodes
    assert r.header.partial_slots > 0
    need = -(-r.header.row_blocks * 4 // 256) * 256 + r.header.partial_slots * 8 * 128 * 4
    assert need <= lib.grb_static_scratch_bytes()
    stream = torch.cuda.current_stream(dev).cuda_stream
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    g = torch.Generator().manual_seed(5)
    for m in (8, 3):                                         # two calls in a row on one stream
        x = torch.randn(m, 4096, generator=g).to(torch.bfloat16).to(dev)
        want = torch.empty(m, 1024, device=dev, dtype=torch.bfloat16)
        r.gemv(x, want)
        got = torch.full((m, 1024), float("nan"), device=dev, dtype=torch.bfloat16)
        st = lib.grb_bxr_gemv_static(r.image.data_ptr(), ctypes.byref(r.header), x.data_ptr(), x.stride(0), m, got.data_ptr(),
                                     got.stride(0), None, status.data_ptr(), stream)
        assert st == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0 and r.check_status() == 0
        assert np.array_equal(got.view(torch.uint16).cpu().numpy(), want.view(torch.uint16).cpu().numpy())
        ref = x.float() @ torch.from_numpy(words.view(np.int16)).view(torch.bfloat16).to(dev).float().T
        assert ((got.float() - ref).abs().max() / ref.abs().max()).item() <= 1e-2   # same tolerance as the other GPU tests


def test_static_scratch_limit_is_refused_without_launching(orc):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from georefine_b200 import _native
    from georefine_b200.resident import build_image

    lib = _native.lib()
    # built for 2048 workers, every 128x128 unit of a 4096 x 5120 weight is its own work item: 1280 shared
    # partial tiles, 5 MiB of GEMV scratch, more than the 4 MiB array holds
    words = orc.synthetic_weight_words(4096, 5120, 42)
    image, h = build_image(words, 2048, layout="rans")
    assert h.partial_slots * 8 * 128 * 4 > lib.grb_static_scratch_bytes()
    dev = torch.device("cuda:0")
    img = torch.from_numpy(image).to(dev)
    x = torch.zeros(1, 5120, device=dev, dtype=torch.bfloat16)
    y = torch.full((1, 4096), 7.0, device=dev, dtype=torch.bfloat16)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    st = lib.grb_bxr_gemv_static(img.data_ptr(), ctypes.byref(h), x.data_ptr(), 5120, 1, y.data_ptr(), 4096, None, status.data_ptr(),
                                 torch.cuda.current_stream(dev).cuda_stream)
    assert st == 4                                           # GRB_ERR_STATIC_LIMIT
    torch.cuda.synchronize()
    assert bool((y == 7.0).all())


def test_static_scratch_gemv_on_the_default_layout(orc):
    """An image in the default 4-bit window layout: the allocation-free entry point then runs the tensor-core kernel at
    its narrowest tile, partial tiles and counters in the library's fixed array.  Two calls in a row, each bit for bit
    what grb_bxr_gemv returns with caller-owned scratch."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from georefine_b200 import _native
    from georefine_b200.resident import ResidentWeight

    lib = _native.lib()
    dev = torch.device("cuda:0")
    words = orc.synthetic_weight_words(1024, 4096, 43)
    r = ResidentWeight.from_words(words, dev, layout="window4")
    assert r.mode == 3 and r.header.partial_slots > 0
    assert -(-r.header.row_blocks * 4 // 256) * 256 + r.header.partial_slots * 16 * 128 * 4 <= lib.grb_static_scratch_bytes()
    stream = torch.cuda.current_stream(dev).cuda_stream
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    g = torch.Generator().manual_seed(6)
    w = torch.from_numpy(words.view(np.int16)).view(torch.bfloat16).to(dev).float()
    for m in (5, 8):
        x = torch.randn(m, 4096, generator=g).to(torch.bfloat16).to(dev)
        want = torch.empty(m, 1024, device=dev, dtype=torch.bfloat16)
        r.gemv(x, want)
        got = torch.full((m, 1024), float("nan"), device=dev, dtype=torch.bfloat16)
        st = lib.grb_bxr_gemv_static(r.image.data_ptr(), ctypes.byref(r.header), x.data_ptr(), x.stride(0), m, got.data_ptr(),
                                     got.stride(0), None, status.data_ptr(), stream)
        assert st == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0 and r.check_status() == 0
        assert np.array_equal(got.view(torch.uint16).cpu().numpy(), want.view(torch.uint16).cpu().numpy())
        ref = x.float() @ w.T
        assert ((got.float() - ref).abs().max() / ref.abs().max()).item() <= 1e-2


def test_static_scratch_gemv_refuses_bad_arguments_before_touching_the_stream(orc):
    """A refused call must leave the output alone and put nothing on the stream: the checks (batch above 8, null or
    misaligned activations, a row stride that is not a multiple of 8) come before the counters are cleared."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from georefine_b200 import _native
    from georefine_b200.resident import ResidentWeight

    lib = _native.lib()
    dev = torch.device("cuda:0")
    r = ResidentWeight.from_words(orc.synthetic_weight_words(256, 512, 44), dev, layout="window4")
    stream = torch.cuda.current_stream(dev).cuda_stream
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    x = torch.zeros(16, 520, device=dev, dtype=torch.bfloat16)
    y = torch.full((16, 256), 7.0, device=dev, dtype=torch.bfloat16)
    call = lambda xp, ldx, m: lib.grb_bxr_gemv_static(r.image.data_ptr(), ctypes.byref(r.header), xp, ldx, m, y.data_ptr(), 256,
                                                      None, status.data_ptr(), stream)
    assert call(x.data_ptr(), 520, 9) == 2            # GRB_ERR_UNSUPPORTED: more than 8 batch rows
    assert call(None, 520, 1) == 1                    # GRB_ERR_ARGUMENT
    assert call(x.data_ptr() + 2, 520, 1) == 1        # activations not 16-byte aligned
    assert call(x.data_ptr(), 515, 1) == 1            # row stride not a multiple of 8 elements
    assert call(x.data_ptr(), 520, 0) == 1
    torch.cuda.synchronize()
    assert bool((y == 7.0).all()) and int(status.item()) == 0
    assert call(x.data_ptr(), 520, 1) == 0            # and a good call still works afterwards
    torch.cuda.synchronize()
    assert bool((y[0] == 0).all()) and int(status.item()) == 0
