"""The allocation-free C entry point for paged decode attention, called through ctypes like a plain C client would.

Collected last on purpose (file name): it must pass alone and after every other test has used the device."""
import ctypes
import math
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    import unirl_b200
    from unirl_b200.ops._ext import require_ext

    require_ext()  # loads the extension (and libtorch) into the process first
    lib = ctypes.CDLL(os.path.join(os.path.dirname(unirl_b200.__file__), "_C.so"))
    fn = lib.unirl_b200_paged_decode_attention_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 7 + [ctypes.c_float, ctypes.c_void_p]
    lib.unirl_b200_decode_noalloc_workspace_floats.restype = ctypes.c_int64
    lib.unirl_b200_decode_noalloc_workspace_floats.argtypes = [ctypes.c_int] * 5
    lib.unirl_b200_decode_noalloc_setup.restype = ctypes.c_int
    return lib


def _case(b, hq, hkv, d, page, max_len, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    lens = torch.randint(max_len // 3, max_len + 1, (b,), generator=g, device="cuda", dtype=torch.int32)
    max_pages = (max_len + page - 1) // page
    n_pages = b * max_pages + 3
    kc = torch.randn(n_pages, hkv, page, d, generator=g, device="cuda").bfloat16()
    vc = torch.randn(n_pages, hkv, page, d, generator=g, device="cuda").bfloat16()
    bt = torch.randperm(n_pages, generator=g, device="cuda")[: b * max_pages].view(b, max_pages).to(torch.int32).contiguous()
    q = torch.randn(b, hq, d, generator=g, device="cuda").bfloat16()
    return q, kc, vc, bt, lens, max_pages


def test_noalloc_decode_attention_matches_regular_entry_point_twice():
    from unirl_b200.ops.attention import paged_decode_attention

    lib = _lib()
    assert lib.unirl_b200_decode_noalloc_setup() == 0
    stream = torch.cuda.current_stream().cuda_stream
    for seed, (b, hq, hkv, d, page, max_len) in enumerate([(6, 32, 8, 128, 32, 700), (3, 16, 4, 64, 16, 300)]):  # two calls in a row share the scratch array
        q, kc, vc, bt, lens, max_pages = _case(b, hq, hkv, d, page, max_len, seed)
        want = paged_decode_attention(q, kc, vc, bt, lens, 1.0 / math.sqrt(d), None, max_len)
        out = torch.full_like(q, float("nan"))
        before = torch.cuda.memory_stats()["allocation.all.allocated"]
        rc = lib.unirl_b200_paged_decode_attention_noalloc(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), lens.data_ptr(), out.data_ptr(), b, hq, hkv,
                                                           d, page, max_pages, max_len, 1.0 / math.sqrt(d), stream)
        assert rc == 0
        assert torch.cuda.memory_stats()["allocation.all.allocated"] == before  # the tensor library's allocator was not touched
        torch.cuda.synchronize()
        torch.testing.assert_close(out.float(), want.float(), atol=2e-2, rtol=2e-2)


def test_noalloc_rejects_oversize_and_bad_shapes():
    lib = _lib()
    need = lib.unirl_b200_decode_noalloc_workspace_floats(256, 64, 1, 128, 65536)
    assert need > 4 * 1024 * 1024
    dummy = torch.zeros(16, device="cuda", dtype=torch.int32)
    p = dummy.data_ptr()
    assert lib.unirl_b200_paged_decode_attention_noalloc(p, p, p, p, p, p, 256, 64, 1, 128, 32, 2048, 65536, 1.0, None) == 3  # too large: refused before any launch
    assert lib.unirl_b200_paged_decode_attention_noalloc(p, p, p, p, p, p, 2, 8, 8, 96, 32, 4, 128, 1.0, None) == 1  # head_dim 96 unsupported
    torch.cuda.synchronize()


def test_noalloc_call_after_setup_can_be_captured_and_replayed():
    """setup() does everything that is per device (scratch address, kernel attributes), so a call made afterwards contains only
    kernel launches: it is recorded into a CUDA graph on a side stream and replayed against fresh inputs."""
    from unirl_b200.ops.attention import paged_decode_attention

    lib = _lib()
    assert lib.unirl_b200_decode_noalloc_setup() == 0
    b, hq, hkv, d, page, max_len = 4, 16, 4, 128, 32, 500
    q, kc, vc, bt, lens, max_pages = _case(b, hq, hkv, d, page, max_len, 7)
    out = torch.zeros_like(q)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        rc = lib.unirl_b200_paged_decode_attention_noalloc(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), lens.data_ptr(), out.data_ptr(), b, hq, hkv,
                                                           d, page, max_pages, max_len, 1.0 / math.sqrt(d), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    q.copy_(torch.randn_like(q))  # the graph reads the same addresses: new contents, same launches
    graph.replay()
    torch.cuda.synchronize()
    want = paged_decode_attention(q, kc, vc, bt, lens, 1.0 / math.sqrt(d), None, max_len)
    torch.testing.assert_close(out.float(), want.float(), atol=2e-2, rtol=2e-2)
