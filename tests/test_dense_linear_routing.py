"""``dense.linear`` / ``install_dense`` on the CPU: which calls may go to the GEMV, and that everything else is plain
``F.linear`` with the reason counted (the reference's ``miv_gemv.linear`` / ``install_dense`` contract,
glc_serve/miv_gemv.py:893-969).  The GEMV route itself needs a GPU (tests/test_gpu_dense_gemv.py)."""
import pytest

torch = pytest.importorskip("torch")
from torch import nn  # noqa: E402

from georefine_b200 import dense  # noqa: E402


def test_cpu_operands_fall_back_and_are_counted():
    dense.STATS.reset()
    w, x, b = torch.randn(6, 16).bfloat16(), torch.randn(2, 3, 16).bfloat16(), torch.randn(6).bfloat16()
    y = dense.linear(x, w, b)
    assert torch.equal(y, torch.nn.functional.linear(x, w, b)) and y.shape == (2, 3, 6)
    assert dense.STATS.fallback_by_reason == {"not_cuda": 1} and dense.STATS.gemv_by_m == {}
    dense.enable(False)
    try:
        dense.linear(x, w)
        assert dense.STATS.fallback_by_reason == {"not_cuda": 1, "disabled": 1}
    finally:
        dense.enable(True)


def test_install_wraps_plain_linears_once():
    dense.STATS.reset()
    class Special(nn.Linear):          # a subclass may have a forward of its own: left alone
        pass

    model = nn.Sequential(nn.Linear(8, 8), nn.ReLU(), nn.Sequential(nn.Linear(8, 4, bias=False), Special(4, 4))).bfloat16()
    x = torch.randn(5, 8).bfloat16()
    want = model(x)
    assert dense.install_dense(model, prefix_filter=["2."]) == 1
    assert dense.install_dense(model) == 1 and dense.install_dense(model) == 0
    assert torch.equal(model(x), want)
    assert dense.STATS.fallback_by_reason == {"not_cuda": 2}


class _Fake:
    """Just enough of a CUDA tensor for the eligibility rules."""

    def __init__(self, shape, dtype=torch.bfloat16, strides=None, ptr=256, cuda=True):
        self.shape, self.dtype, self.is_cuda, self._ptr = tuple(shape), dtype, cuda, ptr
        self._strides = strides or tuple(int(torch.tensor(shape[i + 1:]).prod()) for i in range(len(shape)))

    def dim(self):
        return len(self.shape)

    def stride(self, i):
        return self._strides[i]

    def data_ptr(self):
        return self._ptr

    def numel(self):
        return int(torch.tensor(self.shape).prod())


def test_eligibility_rules():
    w = _Fake((64, 256))
    assert dense.ineligible(_Fake((3, 256)), w) is None
    assert dense.ineligible(_Fake((2, 4, 256)), w) is None
    assert dense.ineligible(_Fake((9, 256)), w) == "m_gt8"
    assert dense.ineligible(_Fake((0, 256)), w) == "m_lt1"
    assert dense.ineligible(_Fake((3, 128)), w) == "shape_mismatch"
    assert dense.ineligible(_Fake((3, 256), dtype=torch.float32), w) == "x_not_bf16"
    assert dense.ineligible(_Fake((3, 256)), _Fake((64, 256), dtype=torch.float16)) == "weight_not_bf16_matrix"
    assert dense.ineligible(_Fake((3, 252)), _Fake((64, 252))) == "k_not_multiple_of_8"
    assert dense.ineligible(_Fake((3, 256)), _Fake((64, 256), strides=(1, 64))) == "weight_layout"
    assert dense.ineligible(_Fake((3, 256)), _Fake((64, 256), ptr=264)) == "weight_layout"
    assert dense.ineligible(_Fake((3, 256), cuda=False), w) == "not_cuda"
