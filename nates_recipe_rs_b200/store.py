"""Python binding of the tiered weight store (include/qmm_store.h): device claim, pinned host memory, file;
the role gpu-core/src/waterfall.rs and the streaming glue of examples/gemma4.rs play upstream."""
import ctypes as C

import numpy as np

from ._lib import StoreStats, check, lib

VRAM, RAM, DISK = 0, 1, 2


class WeightStore:
    def __init__(self, vram_budget=0, ram_budget=0, stage_bytes=0, cache_slots=0, cache_slot_bytes=0):
        self.h = C.c_void_p()
        check(lib().qmm_store_create(vram_budget, ram_budget, stage_bytes, cache_slots, cache_slot_bytes, C.byref(self.h)), "qmm_store_create")

    def close(self):
        if self.h:
            lib().qmm_store_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def place_host(self, name, data):
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        check(lib().qmm_store_place_host(self.h, name.encode(), data.ctypes.data_as(C.c_void_p), data.size), f"qmm_store_place_host({name})")
        return self.home(name)

    def place_file(self, name, path, offset, nbytes):
        check(lib().qmm_store_place_file(self.h, name.encode(), str(path).encode(), offset, nbytes), f"qmm_store_place_file({name})")
        return self.home(name)

    def home(self, name):
        t = lib().qmm_store_home(self.h, name.encode())
        if t < 0:
            check(t, f"qmm_store_home({name})")
        return t

    def stats(self):
        s = StoreStats()
        check(lib().qmm_store_stats(self.h, C.byref(s)), "qmm_store_stats")
        return {n: getattr(s, n) for n, _ in StoreStats._fields_}

    def _stream(self):
        import torch
        return torch.cuda.current_stream().cuda_stream

    def fetch(self, name):
        """Device address (int) of the blob's bytes for work on the current torch stream."""
        p = C.c_void_p()
        check(lib().qmm_store_fetch(self.h, name.encode(), self._stream(), C.byref(p)), f"qmm_store_fetch({name})")
        return p.value

    def prefetch(self, name):
        check(lib().qmm_store_prefetch(self.h, name.encode(), self._stream()), f"qmm_store_prefetch({name})")

    def fetch_cached(self, name):
        p = C.c_void_p()
        check(lib().qmm_store_fetch_cached(self.h, name.encode(), self._stream(), C.byref(p)), f"qmm_store_fetch_cached({name})")
        return p.value
