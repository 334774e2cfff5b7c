"""Operator-graph specs used by the golden fixtures and the parity tests.

One entry per whitelist strategy of the reference's tuner (whilte_list_path_impl.cc: strategies
1-9) plus the two 3-level templates that only the general API reaches. Spec grammar: see
oracle/ref_dump.cc.
"""

COMPRESSED_SPECS = {
    # strategy 1: row_padding -> BLB row div (evenly) -> TLB row div -> SELL-like
    "S1_K2": "sub all row_padding 64 1\nsub all blb_row_evenly 64\nsub all tlb_row\nsub all template K2",
    # strategy 5: row_padding(32) -> TLB row div -> ELL-like
    "S5_K3": "sub all row_padding 32 1\nsub all tlb_row\nsub all template K3",
    # strategy 9: TLB nnz div -> CSR5-like (two templates)
    "S9_K9": "sub all tlb_nnz 4\nsub all template K9",
    "S9_K10": "sub all tlb_nnz 4\nsub all template K10",
    # strategy 4: WLB col div -> warp per row chunk
    "S4_K4": "sub all wlb_col_fixed 32\nsub all template K4",
    # strategies 6 / 7: BLB rows -> WLB col div -> warp partials + smem row reduce
    "S6_K8": "sub all row_padding 4 1\nsub all blb_row_evenly 4\nsub all wlb_col_fixed 32\nsub all template K8",
    "S7_K8": "sub all blb_row_nnz 512\nsub all wlb_col_fixed 32\nsub all template K8",
    # strategies 2 / 3: BLB rows -> TLB col div -> TLB partials + smem row reduce
    "S2_K6": "sub all row_padding 32 1\nsub all blb_row_evenly 32\nsub all tlb_col_fixed 4\nsub all template K6",
    "S3_K6": "sub all blb_row_nnz 512\nsub all tlb_col_fixed 4\nsub all template K6",
    # strategy 8: BLB col div -> CTA per long-row chunk
    "S8_K7": "sub all blb_col_fixed 128\nsub all template K7",
    # general 3-level tilings
    "X_K1": "sub all blb_row_evenly 64\nsub all wlb_row_evenly 16\nsub all tlb_col_fixed 4\nsub all template K1",
    "X_K5": "sub all blb_row_evenly 64\nsub all wlb_row_evenly 16\nsub all tlb_col_fixed 4\nsub all template K5",
}


def full_spec(name: str, dense: str = "dense compress") -> str:
    return dense + "\n" + COMPRESSED_SPECS[name]


# dense-view strategy 3 of the tuner: coarse sort (step 1) -> exponential row division -> compress,
# with a different compressed-view path per strip (long rows first: the sort is descending)
SORTED_SPLIT_SPEC = """dense sort 1
dense rowdiv_exp 32 4096 4
dense compress
sub 0 blb_col_fixed 128
sub 0 template K7
sub 1 row_padding 32 1
sub 1 blb_row_evenly 32
sub 1 tlb_col_fixed 4
sub 1 template K6
sub 2 row_padding 32 1
sub 2 blb_row_evenly 32
sub 2 tlb_row
sub 2 template K2
sub 3 row_padding 32 1
sub 3 tlb_row
sub 3 template K3"""

# dense-view strategy 2: exponential row division without sort
SPLIT_SPEC = """dense rowdiv_exp 32 4096 4
dense compress
sub all row_padding 32 1
sub all blb_row_evenly 32
sub all tlb_col_fixed 2
sub all template K6"""
