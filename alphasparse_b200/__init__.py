"""B200-native SpMV over AlphaSparse's machine-designed formats.

`capi` binds the device side of the C ABI of `libasp_b200.so` (include/asp_b200.h), `graph` the host
side (include/asp_b200_host.h: matrices, Operator Graphs, lowered formats, the search loop), `tuner`
is the search as Python sees it, `dist` shards a matrix over the GPUs of a node, `matrices` and
`matrices_gpu` hold the seeded synthetic inputs. There is no CPU fallback: using `capi` without the
built library raises.
"""
