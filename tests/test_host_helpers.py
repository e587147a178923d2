"""Host-side helpers of the exchange and of the chunked preprocess launches (pure integer logic, no GPU)."""
import numpy as np
import pytest

import util  # noqa: F401
from cgx import exchange as EX
from cgx.batched import chunk_bounds


@pytest.mark.parametrize("P,chunks", [(0, 4), (1, 4), (255, 2), (256, 4), (257, 2), (1000, 3), (750_000, 4),
                                      (6_000_000, 4), (6_000_000, 1), (513, 100)])
def test_chunk_bounds_cover_the_range_in_whole_ctas(P, chunks):
    b = chunk_bounds(P, chunks)
    assert b[0][0] == 0 and b[-1][1] == P
    assert len(b) <= max(1, chunks)
    for (lo, hi), (lo2, _) in zip(b, b[1:]):
        assert hi == lo2                               # contiguous
    for lo, hi in b:
        assert lo % 256 == 0 and (hi > lo or P == 0)   # whole CTAs, 16-byte aligned row offsets for every width


def test_camera_layouts_align_every_tensor():
    n = np.array([[0, 1, 7], [1000, 333, 12345]])
    for fields in (EX._CAM_FIELDS, EX._CAM_FIELDS_PLANES):
        offs, size = EX._camera_layouts(n, fields)
        assert offs.shape == n.shape + (len(fields),) and size.shape == n.shape
        assert (offs % 256 == 0).all() and (size % 256 == 0).all()
        widths = np.array([w for _, w in fields])
        ends = offs + n[..., None] * widths
        assert (ends[..., :-1] <= offs[..., 1:]).all() and (ends[..., -1] <= size).all()
    assert EX._camera_layout(0) == ([0] * 8, 0)


def test_destination_rows_are_padded_to_the_struct_width():
    t9 = np.arange(18, dtype=np.uint64).reshape(2, 9)
    t10 = EX._dst_rows(t9, 2)
    assert t10.shape == (2, 10) and t10.flags["C_CONTIGUOUS"] and t10.dtype == np.uint64
    assert (t10[:, :9] == t9).all() and (t10[:, 9] == 0).all()
    assert EX._dst_rows(t10, 2) is not None
    with pytest.raises(AssertionError):
        EX._dst_rows(t9, 3)
