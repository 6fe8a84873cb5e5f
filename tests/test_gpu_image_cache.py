"""A linear served from the verified image cache: second load hits, skips the host walk, and multiplies the same bits."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def test_cached_linear_hits_on_the_second_load_and_matches(tmp_path, orc):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from georefine_b200 import codec, image_cache

    dev = torch.device("cuda:0")
    words = orc.synthetic_weight_words(384, 640, 55)
    frame = codec.encode(words)
    cache = image_cache.ImageCache(tmp_path, verify="full")
    first = image_cache.CachedLinear(frame, device=dev, cache=cache)
    second = image_cache.CachedLinear(frame, device=dev, cache=cache)
    assert not first.cache_hit and second.cache_hit and cache.stats == {**cache.stats, "hits": 1, "writes": 1}
    assert second.shape == words.shape and second.source_sha256 == first.source_sha256 and second.frame_bytes == len(frame)
    got = second.decode().view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, words)
    x = torch.randn(5, 640, device=dev).to(torch.bfloat16)
    ya, yb = first.linear(x), second.linear(x)
    ref = x.float() @ torch.from_numpy(words.view(np.int16)).view(torch.bfloat16).to(dev).float().T
    assert torch.equal(ya, yb) and ((yb.float() - ref).abs().max() / ref.abs().max()).item() <= 1e-2   # BF16 out, FP32 accumulate
    ids = torch.tensor([0, 383, 17], device=dev)
    assert np.array_equal(second.gather_rows(ids).view(torch.int16).cpu().numpy().view(np.uint16), words[[0, 383, 17]])
