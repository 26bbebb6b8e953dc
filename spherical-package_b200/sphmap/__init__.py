"""Python-side helpers around the C ABI of libsphmap.so: a ctypes binding
(``capi``), the seeded synthetic workloads used for parity and measurement
(``workloads``) and the batch-sharded data-parallel helpers (``parallel``)."""
