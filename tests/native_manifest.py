"""Adapter (test infrastructure): presents a natively lowered Format the way plan_interp expects a
reference manifest, so that the CPU suite can compute y from the native arrays without a GPU."""
from alphasparse_b200 import capi

_TEMPLATE_NAME = {v: k for k, v in capi.TEMPLATE.items()}


class NativeManifest:
    def __init__(self, fmt, n_rows: int):
        self.fmt = fmt
        self.meta = {"rows": int(n_rows)}
        self.subs = []
        for d in fmt.plan_descs():
            sub = {
                "template": _TEMPLATE_NAME[d.template_type], "first_row": int(d.first_row), "first_col": int(d.first_col),
                "global_sort": d.sort_kind == capi.SORT_GLOBAL, "local_sort": d.sort_kind == capi.SORT_LOCAL,
                "thread_block_size_in_block": int(d.tlb_size), "tlb_size": int(d.tlb_size),
                "bits_word": int(d.bits_word), "bits_flag": int(d.bits_flag), "bits_row": int(d.bits_row), "bits_off": int(d.bits_off),
            }
            if d.effective_num:  # 0 = the template has no effective count (every unit is live)
                sub.update({"effective_TLB_num": int(d.effective_num), "effective_WLB_num": int(d.effective_num), "effective_row_num": int(d.effective_num)})
            self.subs.append(sub)

    def sub_arrays(self, i):
        return {name: (arr, comp, {"len": ln}) for name, (arr, comp, dt, ln) in self.fmt.arrays(i).items()}
