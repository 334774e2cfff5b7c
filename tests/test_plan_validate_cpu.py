"""CPU suite: asp_plan_descs_validate, the host-only half of asp_plan_group_create.

What a caller hands over is checked before any kernel can read it: every column index inside x,
every row a kernel can write inside y, every offset inside the array it indexes. The reference
asserts on malformed template structs (or, compiled with -DNDEBUG, reads past its arrays); here a
bad array is a status and a message, and it never reaches a GPU that other jobs share.
"""
import ctypes as C

import numpy as np
import pytest

import refdump
import specs
from alphasparse_b200 import capi, matrices as M
from alphasparse_b200.graph import Format, Matrix
from golden_util import golden_names, load_golden

BOUNDS = 5  # ASP_ERR_BOUNDS


@pytest.mark.parametrize("name", golden_names())
def test_reference_built_arrays_validate(name):
    _, _, _, man = load_golden(name)
    descs, keep = refdump.plan_descs(man)
    capi.validate_descs(descs)


def _array_of(desc, role_name):
    """(index, numpy view) of the array with this role in a plan descriptor; the view aliases the
    host buffer the descriptor points at, so writing through it corrupts what validation sees."""
    role = capi.ROLE[role_name]
    np_of = {capi.U8: np.uint8, capi.U16: np.uint16, capi.U32: np.uint32, capi.U64: np.uint64}
    for k in range(desc.n_arrays):
        a = desc.arrays[k]
        if a.role == role and a.compress == 0 and a.host_ptr:
            dt = np.dtype(np_of[a.dtype])
            buf = (C.c_uint8 * (a.len * dt.itemsize)).from_address(a.host_ptr)
            return k, np.frombuffer(buf, dtype=dt)
    return None, None


def _expect_bounds(descs, needle):
    with pytest.raises(capi.AspError) as e:
        capi.validate_descs(descs)
    assert e.value.status == BOUNDS, str(e.value)
    assert needle in str(e.value), str(e.value)


# one fixture per kernel family, and the array whose largest entry names a row
ROW_ARRAYS = [
    ("uniform1024_f32_S5_K3", "global_row_index_of_thread_level_block"),
    ("uniform1024_f32_S1_K2", "global_row_index_of_thread_level_block"),
    ("uniform1024_f32_X_K1", "global_row_index_of_thread_level_block"),
    ("uniform1024_f32_S4_K4", "global_row_index_of_warp_level_block"),
    ("uniform1024_f32_S8_K7", "row_index_of_block_level_block"),
    ("uniform1024_f32_S9_K9", "global_first_row_index_of_warp_level_block"),
    ("uniform1024_f32_S9_K10", "global_first_row_index_of_warp_level_block"),
]


@pytest.mark.parametrize("name", sorted({n for n, _ in ROW_ARRAYS} | {"uniform1024_f32_S2_K6", "uniform1024_f32_S6_K8", "uniform1024_f32_X_K5", "fem128_f64_S5_K3"}))
def test_a_column_outside_x_is_rejected(name):
    m, _, _, man = load_golden(name)
    descs, keep = refdump.plan_descs(man)
    _, col = _array_of(descs[0], "col_index_arr")
    old = col[len(col) // 2]
    if np.iinfo(col.dtype).max < m.n_cols:
        # the narrowed type cannot even express a column outside x: declare a smaller x instead
        descs[0].n_cols = int(col.max())
    else:
        col[len(col) // 2] = m.n_cols
    _expect_bounds(descs, "column outside x")
    col[len(col) // 2] = old


@pytest.mark.parametrize("name,role", ROW_ARRAYS)
def test_a_row_outside_y_is_rejected(name, role):
    m, _, _, man = load_golden(name)
    descs, keep = refdump.plan_descs(man)
    k, rows = _array_of(descs[0], role)
    if rows is None:
        # the reference replaced the array by a closed form: push the closed form out of range instead
        r = capi.ROLE[role]
        for j in range(descs[0].n_arrays):
            if descs[0].arrays[j].role == r:
                descs[0].arrays[j].icpt += m.n_rows
        _expect_bounds(descs, "outside y") if "first_row" not in role else _expect_bounds(descs, "")
        return
    if np.iinfo(rows.dtype).max < m.n_rows:
        descs[0].n_rows = int(rows.max())  # y shorter than the largest row named
        if descs[0].first_row >= descs[0].n_rows:
            pytest.skip("first_row check fires first")
    else:
        rows[0] = m.n_rows + 3
    with pytest.raises(capi.AspError) as e:
        capi.validate_descs(descs)
    assert e.value.status == BOUNDS


@pytest.mark.parametrize("name", ["uniform1024_f32_S2_K6", "uniform1024_f32_S6_K8", "uniform1024_f32_S7_K8", "uniform1024_f32_X_K5"])
def test_partial_result_offsets_must_stay_inside_their_blb(name):
    _, _, _, man = load_golden(name)
    descs, keep = refdump.plan_descs(man)
    role = "row_offset_in_warp_tmp_result" if name.endswith("K8") else "row_offset_in_thread_tmp_result"
    _, off = _array_of(descs[0], role)
    if off is not None:
        off[1] = np.iinfo(off.dtype).max  # row 0 now claims partial results far past its BLB's shared memory
    else:
        # the reference replaced the offsets by a closed form (equal rows): stretch it
        for j in range(descs[0].n_arrays):
            if descs[0].arrays[j].role == capi.ROLE[role]:
                assert descs[0].arrays[j].compress == capi.COMPRESS["linear"]
                descs[0].arrays[j].coef *= 1000
    _expect_bounds(descs, "partial-result range")


def test_sorted_plan_with_a_bad_permutation_is_rejected():
    _, _, _, man = load_golden("mixed4096_f32_sorted_split")
    descs, keep = refdump.plan_descs(man)
    capi.validate_descs(descs)
    hit = False
    for d in descs:
        _, perm = _array_of(d, "row_index_before_sort")
        if perm is not None and d.template_type in (capi.TEMPLATE["K6"], capi.TEMPLATE["K8"], capi.TEMPLATE["K9"], capi.TEMPLATE["K10"], capi.TEMPLATE["K5"]):
            perm[3] = np.iinfo(perm.dtype).max
            hit = True
            break
    if not hit:
        pytest.skip("no device-permuted strip in this fixture")
    _expect_bounds(descs, "row_index_before_sort")


@pytest.mark.parametrize("spec,dense", [("S5_K3", "dense compress"), ("S9_K9", "dense compress"), ("S2_K6", "dense sort 1\ndense compress"),
                                        ("S1_K2", "dense sort 1\ndense rowdiv_exp 32 4096 4\ndense compress")])
def test_native_formats_validate_and_empty_strips_keep_their_value_type(spec, dense):
    m, _ = M.rmat(10, 6, seed=4)
    m64 = M.CsrMatrix(m.n_rows, m.n_cols, m.indptr, m.indices, m.values.astype(np.float64))
    fmt = Matrix.from_csr(m64).execute(specs.full_spec(spec, dense))
    capi.validate_descs(fmt.plan_descs())
    fmt.close()


def test_a_damaged_format_file_is_rejected_by_loader_or_validation(tmp_path):
    m, _ = M.uniform_random(300, 6, seed=1)
    fmt = Matrix.from_csr(m).execute(specs.full_spec("S5_K3"))
    good = tmp_path / "good.asp"
    fmt.save(str(good))
    data = bytearray(good.read_bytes())
    # 1. flip the element type of the first array record to an undefined one: the loader refuses
    head = 8 + 4 + 4 + 8 * 4  # magic, two i32, four u64
    rec = data.find(bytes(fmt_sub_scalars_prefix(fmt)), head)
    assert rec >= 0
    bad = tmp_path / "bad_dtype.asp"
    corrupt = bytearray(data)
    # the array head follows the sub-matrix scalars, the asp_sub_info and the array count
    arr0 = rec + SUBSCALARS_BYTES + SUBINFO_BYTES + 8
    corrupt[arr0 + 4 : arr0 + 8] = (77).to_bytes(4, "little")
    bad.write_bytes(bytes(corrupt))
    with pytest.raises(capi.AspError):
        Format.load(str(bad))
    # 2. a payload length that disagrees with len * element size: refused
    corrupt = bytearray(data)
    plen = arr0 + 6 * 4 + 4 * 8  # payload_bytes field of the array head
    corrupt[plen : plen + 8] = (3).to_bytes(8, "little")
    bad2 = tmp_path / "bad_payload.asp"
    bad2.write_bytes(bytes(corrupt))
    with pytest.raises(capi.AspError):
        Format.load(str(bad2))
    # 3. an index that points outside x passes the loader (it is structurally sound) and is caught by validation
    back = Format.load(str(good))
    descs = back.plan_descs()
    _, col = _array_of(descs[0], "col_index_arr")
    col[0] = np.iinfo(col.dtype).max
    descs[0].n_cols = min(int(descs[0].n_cols), int(np.iinfo(col.dtype).max))
    _expect_bounds(descs, "column outside x")
    back.close()
    fmt.close()


SUBSCALARS_BYTES = 8 * 4 + 8 * 8 + 3 * 8
SUBINFO_BYTES = 9 * 8 + 2 * 4


def fmt_sub_scalars_prefix(fmt):
    """First bytes of the SubScalars record of sub-matrix 0 (template_type, val_dt as two i32)."""
    d = fmt.plan_descs()[0]
    return int(d.template_type).to_bytes(4, "little") + int(d.val_dtype).to_bytes(4, "little")
