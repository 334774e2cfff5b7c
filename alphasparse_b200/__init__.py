"""B200-native SpMV over AlphaSparse's machine-designed formats.

`capi` binds the C ABI of `libasp_b200.so` (include/asp_b200.h); `matrices` holds the seeded
synthetic inputs. There is no CPU fallback: importing `capi` without the built library raises.
"""
