"""CPU-side checks of the C-ABI boundary: the library loads, exports every symbol the header
declares, and validates arguments before touching a device."""
import ctypes
import pathlib
import re

ROOT = pathlib.Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "bitsknn.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bitsknn_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(bk):
    assert declared_symbols() == sorted(bk.SIGNATURES)


def test_every_declared_symbol_is_exported(bk):
    handle = ctypes.CDLL(str(bk.LIB_PATH))
    for name in declared_symbols():
        assert hasattr(handle, name), name


def test_version_and_error_string(bk):
    assert bk.lib().bitsknn_version() >= 100
    assert isinstance(bk.last_error(), str)


def test_argument_validation_needs_no_device(bk):
    lib = bk.lib()
    fake = ctypes.c_void_p(256)
    # null matrix
    assert lib.bitsknn_select(None, 8, None, 0, None, 1, 8, 1, fake, fake, None) == bk.ERR_INVALID_ARGUMENT
    # k outside 1..2048: the reference's "Unsupported k value"
    assert lib.bitsknn_select(fake, 8, None, 0, None, 1, 8, 0, fake, fake, None) == bk.ERR_UNSUPPORTED_K
    assert "Unsupported k value: 0" in bk.last_error()
    assert lib.bitsknn_select(fake, 8, None, 0, None, 1, 8, 4096, fake, fake, None) == bk.ERR_UNSUPPORTED_K
    # leading dimension shorter than the row
    assert lib.bitsknn_select(fake, 4, None, 0, None, 1, 8, 1, fake, fake, None) == bk.ERR_INVALID_ARGUMENT
    # misaligned matrix
    assert lib.bitsknn_select(ctypes.c_void_p(258), 8, None, 0, None, 1, 8, 1, fake, fake, None) == bk.ERR_INVALID_ARGUMENT
    # merge: too many candidates
    assert lib.bitsknn_merge(fake, fake, 0, 0, 1, 64, 2048, fake, fake, None) == bk.ERR_INVALID_ARGUMENT
    # split: workspace too small
    assert lib.bitsknn_select_split(fake, 8, None, 1, 8, 2, 2, fake, 1, fake, fake, None) == bk.ERR_WORKSPACE
    assert bk.select_split_workspace_bytes(10, 32, 4) == 10 * 4 * 32 * 8


def test_tuning_registry(bk):
    old = bk.get_tuning("select.stages")
    assert old == 0                                   # automatic by default
    bk.set_tuning("select.stages", 3)
    assert bk.get_tuning("select.stages") == 3
    bk.set_tuning("select.stages", old)
    try:
        bk.set_tuning("select.stages", 99)
    except bk.BitsKnnError as err:
        assert err.status == bk.ERR_INVALID_ARGUMENT
    else:
        raise AssertionError("out-of-range tuning value accepted")
    try:
        bk.set_tuning("no.such.key", 1)
    except bk.BitsKnnError as err:
        assert err.status == bk.ERR_INVALID_ARGUMENT
    else:
        raise AssertionError("unknown tuning key accepted")


def test_every_tuning_key_is_documented_in_the_header(bk):
    header = (ROOT / "include" / "bitsknn.h").read_text()
    keys = bk.tuning_keys()
    assert keys, "no tuning keys registered"
    for key in keys:
        assert f'"{key}"' in header, key


def test_tuning_values_that_do_not_exist_are_rejected(bk):
    for bad in (1, 3):
        try:
            bk.set_tuning("select.unroll", bad)
        except bk.BitsKnnError as err:
            assert err.status == bk.ERR_INVALID_ARGUMENT
        else:
            raise AssertionError("select.unroll accepted a value without a kernel")
    assert bk.get_tuning("select.unroll") == 0


def test_more_row_slices_than_a_grid_holds_are_rejected(bk):
    lib = bk.lib()
    fake = ctypes.c_void_p(256)
    # q * splits = 2^31: beyond the grid limit; the workspace claim is large enough, so only the limit can refuse
    rc = lib.bitsknn_select_split(fake, 8, None, 1 << 20, 8, 1, 2048, fake, 1 << 62, fake, fake, None)
    assert rc == bk.ERR_INVALID_ARGUMENT and "grid limit" in bk.last_error()


def test_sharded_entry_points_validate_before_touching_a_device(bk):
    lib = bk.lib()
    handle = ctypes.c_void_p()
    assert lib.bitsknn_sharded_create(ctypes.byref(handle), None, 3, 2) == bk.ERR_INVALID_ARGUMENT
    assert lib.bitsknn_sharded_init(ctypes.byref(handle), None, 0, 0) == bk.ERR_INVALID_ARGUMENT
    assert lib.bitsknn_sharded_workspace_bytes(None, 10, 10) == 0
    assert lib.bitsknn_sharded_destroy(None) == bk.OK
