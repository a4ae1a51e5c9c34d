"""The allocation-free routing-layout entry point, called the way a C host would call it.

Some users of this library cannot allocate device memory while they run: a serving engine
that pre-plans one memory pool and must not grow it, a plugin living in a process whose
allocator it does not own, a plain C program linking the library without torch.  For them
the library exports ``afdep_route_layout_noalloc``: same result as ``route_layout``, but the
cross-CTA scratch is a fixed array inside the library instead of memory requested per call.

This test loads the shared library with ctypes, passes raw device pointers, and checks two
calls in a row against the ordinary (allocating) entry point.  The second call reuses the
array with whatever the first one left in it, which is exactly what the entry point has to
cope with.  Sizes beyond the built-in maximum must be refused with a clear message.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _library():
    from afdep_b200 import _native

    _native.load_native()            # builds if needed and pulls in libtorch's dependencies
    lib = ctypes.CDLL(str(_native.library_path()))
    fn = lib.afdep_route_layout_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 5
    err = lib.afdep_route_layout_noalloc_error
    err.restype = ctypes.c_char_p
    return fn, err


def _call(fn, ids, experts, ffn):
    tokens, top_k = ids.shape
    dev = ids.device
    route_e = torch.full((tokens, top_k), -7, dtype=torch.int32, device=dev)
    route_pos = torch.full((tokens, top_k), -7, dtype=torch.int32, device=dev)
    tok_slot = torch.full((tokens, ffn), -7, dtype=torch.int32, device=dev)
    counts = torch.full((ffn + experts,), -7, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(ids.data_ptr(), tokens, top_k, experts, ffn, route_e.data_ptr(), route_pos.data_ptr(), tok_slot.data_ptr(),
            counts.data_ptr(), stream)
    return rc, (route_e, route_pos, tok_slot, counts)


def test_no_alloc_entry_point_matches_route_layout_twice():
    from afdep_b200.ops.route_layout import route_layout
    from afdep_b200.utils import synthetic

    fn, err = _library()
    torch.cuda.set_device(0)
    cases = [(700, 256, 8, 8), (333, 64, 4, 6)]     # second call: other shape, same scratch array
    for call, (tokens, experts, ffn, top_k) in enumerate(cases):
        gen = torch.Generator().manual_seed(11 + call)
        ids = synthetic.distinct_routes(tokens, experts, top_k, gen)
        ids = torch.where(torch.rand(ids.shape, generator=gen) < 0.1, torch.full_like(ids, -1), ids)
        ids[3, 0] = experts + 1                      # an illegal token, handled the same way by both
        ids = ids.cuda()
        want = route_layout(ids, experts, ffn)
        torch.cuda.synchronize()
        rc, got = _call(fn, ids, experts, ffn)
        assert rc == 0, err().decode()
        torch.cuda.synchronize()
        for name, g, w in zip(("route_e", "route_pos", "tok_slot", "counts"), got, want):
            assert torch.equal(g, w), f"call {call}: {name} differs from route_layout"
        route_e, _, tok_slot, counts = got
        # the two outcomes that no return code reports: the illegal token comes back blanked,
        # and counts of -1 would mean the launch gave up on its wait between CTAs
        assert bool((route_e[3] == -1).all()) and bool((tok_slot[3] == -1).all())
        assert bool((counts >= 0).all())


def test_no_alloc_entry_point_rejects_oversized_requests():
    fn, err = _library()
    torch.cuda.set_device(0)
    ids = torch.zeros((4, 2), dtype=torch.int64, device="cuda")
    rc, _ = _call(fn, ids, 512, 8)                   # more experts than the built-in scratch holds
    assert rc == 2
    assert "256 experts" in err().decode()
    rc, _ = _call(fn, ids, 10, 3)                    # experts do not divide over the ranks
    assert rc == 1
