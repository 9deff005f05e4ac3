"""The split-KV scratch of the MLA decode kernel under CUDA-graph capture order (host logic only, CPU tensors).

A captured launch keeps the scratch addresses it was given.  The slot count rows x head-groups x splits is not
monotone in the batch size, so walking the buckets largest-first can ask for more slots at a smaller bucket."""
import torch

from batchgen_b200.ops import mla_kernel
from batchgen_b200.runtime.graphs import generate_buckets


def _walk(top, n_buckets, H, max_tiles, sms=148):
    return [(b, mla_kernel.decode_slots(b, H, max_tiles, sms)) for b in
            sorted(generate_buckets(top, n_buckets), reverse=True)]


def test_slot_count_is_not_monotone_in_batch():
    walk = _walk(384, 16, 16, 64)
    slots = [s for _, s in walk]
    assert any(later > earlier for earlier, later in zip(slots, slots[1:])), walk


def test_reserved_scratch_never_moves_over_capture_order():
    mla_kernel._SCRATCH.clear()
    mla_kernel._RETIRED.clear()
    for top in (384, 128, 96):
        mla_kernel._SCRATCH.clear()
        buckets = generate_buckets(top, 16)
        need = mla_kernel.reserve_decode_scratch("cpu", buckets, 16, 64, 148)
        base = mla_kernel._scratch("cpu", 1, 16)
        assert base[0].shape[0] >= need
        for b in sorted(buckets, reverse=True):
            cur = mla_kernel._scratch("cpu", mla_kernel.decode_slots(b, 16, 64, 148), 16)
            assert cur[0].data_ptr() == base[0].data_ptr() and cur[1].data_ptr() == base[1].data_ptr(), (top, b)
    assert not mla_kernel._RETIRED


def test_outgrown_scratch_stays_alive():
    """Without the reservation a buffer can be outgrown; the old one must stay allocated for graphs that hold it."""
    mla_kernel._SCRATCH.clear()
    mla_kernel._RETIRED.clear()
    seen = []
    for b, slots in _walk(2048, 16, 16, 256):
        seen.append(mla_kernel._scratch("cpu", slots, 16))
    ptrs = {t[0].data_ptr() for t in seen}
    alive = {t[0].data_ptr() for t in mla_kernel._RETIRED} | {mla_kernel._SCRATCH[("cpu", 16)][0].data_ptr()}
    assert ptrs <= alive
    mla_kernel._SCRATCH.clear()
    mla_kernel._RETIRED.clear()
