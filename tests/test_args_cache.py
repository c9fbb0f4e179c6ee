"""The shims remember validated arguments per input tuple; these tests pin what makes a remembered entry stale.
They run on CPU tensors: only the bookkeeping is exercised, no kernel is called."""
import torch

from eval_test_b200 import _args
from eval_test_b200 import nvfp4_grouped_gemm as G


def _tuple():
    a = torch.zeros((4, 8, 1), dtype=torch.uint8)
    b = torch.zeros((4, 8, 1), dtype=torch.uint8)
    c = torch.zeros((4, 4, 1), dtype=torch.float16)
    return (a, b, c)


def test_entry_is_reused_for_the_same_tensors_only():
    data = _tuple()
    assert _args.lookup(data, data) is None
    ent = _args.remember(data, data, ("args",))
    assert _args.lookup(data, data) is ent


def test_a_different_view_over_the_same_storage_is_not_a_hit():
    """Same tuple object id is impossible to force, so the entry is looked up through the same tuple with one
    tensor swapped for another view that starts at the same address."""
    a, b, c = _tuple()
    data = [a, b, c]
    _args.remember(data, data, ("args",))
    data[0] = a.view(8, 4, 1)                       # same data_ptr, other shape: must be validated afresh
    assert data[0].data_ptr() == a.data_ptr()
    assert _args.lookup(data, data) is None


def test_a_dead_output_tensor_is_not_a_hit():
    a, b, c = _tuple()
    data = [a, b, c]
    _args.remember(data, data, ("args",))
    ptr = c.data_ptr()
    del c
    data[2] = torch.zeros((4, 4, 1), dtype=torch.float16)
    assert _args.lookup(data, data) is None or data[2].data_ptr() != ptr


def test_grouped_fingerprint_covers_scales_and_sizes():
    a, b, c = _tuple()
    sfa, sfb = torch.zeros(16, dtype=torch.uint8), torch.zeros(16, dtype=torch.uint8)
    abc, sfs, sizes = [(a, b, c)], [(sfa, sfb)], [(4, 4, 16, 1)]
    fp = G._fingerprint(abc, sfs, sizes)
    assert fp == G._fingerprint(abc, sfs, sizes)
    other_scale = [(torch.zeros(16, dtype=torch.uint8), sfb)]
    assert G._fingerprint(abc, other_scale, sizes) != fp         # a scale tensor replaced in place
    assert G._fingerprint(abc, sfs, [(4, 4, 32, 1)]) != fp       # sizes changed
    other_abc = [(a, torch.zeros((4, 8, 1), dtype=torch.uint8), c)]
    assert G._fingerprint(other_abc, sfs, sizes) != fp


def test_grouped_cache_holds_no_strong_references():
    import gc
    import weakref
    a, b, c = _tuple()
    ref = weakref.ref(c)
    G._CACHE[12345] = (weakref.ref(c), G._fingerprint([(a, b, c)], [], []), object())
    del a, b, c
    gc.collect()
    assert ref() is None
    G._CACHE.pop(12345)
