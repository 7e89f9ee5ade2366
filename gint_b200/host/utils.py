"""Small host helpers with the reference's names (``gint/host/utils.py``)."""
from __future__ import annotations


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


def fill_tensor_info(ti, input_infos, slot_offset: int = 0) -> None:
    """Write ``ProgramTensorInfo`` records into a 608-byte descriptor block.

    Batch dims are stored innermost-first and padded with stride 0 / shape 1, as the device-side decode expects
    (reference: ``gint/host/utils.py:6-27``, consumer ``load_tensor_infos.py:34-39``).
    """
    for i, t in enumerate(input_infos):
        s = slot_offset + i
        if len(t.batch_strides) != len(t.batch_shape) or len(t.batch_shape) > 4:
            raise ValueError("At most 4 batch axes supported, with one stride per axis")
        ti.elm_size[s] = t.elm_size
        strides = list(reversed(t.batch_strides)) + [0] * (4 - len(t.batch_strides))
        shape = list(reversed(t.batch_shape)) + [1] * (4 - len(t.batch_shape))
        for j in range(4):
            ti.batch_strides[s][j] = strides[j]
            ti.batch_shape[s][j] = shape[j]
        for field in ("block_shape_stride_1", "block_shape_stride_2", "block_grid_dims", "block_grid_steps"):
            src = getattr(t, field)
            dst = getattr(ti, field)[s]
            dst[0], dst[1] = src[0], src[1]
