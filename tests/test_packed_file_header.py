"""Packed candidate file header parsing without a GPU (``manta_b200_packed_file_info``): a hand-written file in the
documented layout is accepted, damaged ones are refused with a reason."""
import struct

import pytest

from manta_b200 import native

LAYOUT_Q8 = native.LAYOUTS["q8"]


def _header(layout, rows, cols, elem_row_bytes, scale_row_bytes, data_offset, scales_offset, row_base=0, magic=b"MB2PACK\0",
            version=1):
    h = struct.pack("<8sIIqiiiiqqqQ", magic, version, layout, rows, cols, elem_row_bytes, scale_row_bytes, 0, data_offset,
                    scales_offset, row_base, 0)
    return h + b"\0" * (256 - len(h))


def _write(path, header, payload_bytes):
    with open(path, "wb") as f:
        f.write(header)
        f.write(b"\x01" * payload_bytes)


def test_well_formed_q8_file(tmp_path):
    rows, cols = 10, 100
    data_off, scales_off = 256, 256 + 1024  # codes 1000 B, padded to the next multiple of 256
    p = str(tmp_path / "ok.mb2")
    _write(p, _header(LAYOUT_Q8, rows, cols, cols, 4, data_off, scales_off, row_base=77), 1024 + rows * 4)
    info = native.packed_file_info(p)
    assert info == {"layout": LAYOUT_Q8, "rows": rows, "cols": cols, "row_base": 77, "stored_bytes": rows * (cols + 4)}


@pytest.mark.parametrize("what,kwargs,match", [
    ("magic", dict(magic=b"NOTMAGIC"), "not a packed candidate file"),
    ("version", dict(version=9), "unsupported version 9"),
])
def test_bad_identification(tmp_path, what, kwargs, match):
    p = str(tmp_path / (what + ".mb2"))
    _write(p, _header(LAYOUT_Q8, 10, 100, 100, 4, 256, 1280, **kwargs), 2000)
    with pytest.raises(native.MantaError, match=match):
        native.packed_file_info(p)


def test_inconsistent_geometry_and_truncation(tmp_path):
    p = str(tmp_path / "geom.mb2")
    _write(p, _header(LAYOUT_Q8, 10, 100, 99, 4, 256, 1280), 2000)  # q8 stores cols bytes per row, not 99
    with pytest.raises(native.MantaError, match="geometry is inconsistent"):
        native.packed_file_info(p)
    p = str(tmp_path / "short.mb2")
    _write(p, _header(LAYOUT_Q8, 10, 100, 100, 4, 256, 1280), 1024 + 20)  # scales section cut off
    with pytest.raises(native.MantaError, match="sections exceed the file"):
        native.packed_file_info(p)
    p = str(tmp_path / "tiny.mb2")
    open(p, "wb").write(b"MB2PACK\0")
    with pytest.raises(native.MantaError, match="shorter than its header"):
        native.packed_file_info(p)


def test_huge_row_count_and_bad_row_base_are_refused(tmp_path):
    # a row count whose products with the row sizes wrap 64 bits must not pass the bounds check
    p = str(tmp_path / "wrap.mb2")
    _write(p, _header(LAYOUT_Q8, (1 << 62) + 10, 100, 100, 4, 256, 1280), 2000)
    with pytest.raises(native.MantaError, match="sections exceed the file"):
        native.packed_file_info(p)
    p = str(tmp_path / "neg_base.mb2")
    _write(p, _header(LAYOUT_Q8, 10, 100, 100, 4, 256, 1280, row_base=-1), 1024 + 40)
    with pytest.raises(native.MantaError, match="do not fit int32"):
        native.packed_file_info(p)
    p = str(tmp_path / "big_base.mb2")
    _write(p, _header(LAYOUT_Q8, 10, 100, 100, 4, 256, 1280, row_base=2**31 - 5), 1024 + 40)
    with pytest.raises(native.MantaError, match="do not fit int32"):
        native.packed_file_info(p)
