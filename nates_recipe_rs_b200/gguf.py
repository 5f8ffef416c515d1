"""Python binding of the GGUF reader and writer (include/qmm_gguf.h): the weight-file side of the quantized
path, in the role recipe-infer/src/safetensors.rs plays upstream (header-only parse, tensors on demand)."""
import ctypes as C

import numpy as np

from ._lib import GgufTensorInfo, check, lib

F32, F16 = 0, 1


class GgufFile:
    def __init__(self, path):
        self.h = C.c_void_p()
        check(lib().qmm_gguf_open(str(path).encode(), C.byref(self.h)), f"qmm_gguf_open({path})")

    def close(self):
        if self.h:
            lib().qmm_gguf_close(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def __len__(self):
        return lib().qmm_gguf_tensor_count(self.h)

    def info(self, index):
        t = GgufTensorInfo()
        check(lib().qmm_gguf_tensor_info(self.h, index, C.byref(t)), "qmm_gguf_tensor_info")
        return {"name": t.name.decode(), "type": t.type, "dims": list(t.dims)[:t.n_dims], "file_offset": t.file_offset, "bytes": t.bytes}

    def find(self, name):
        return lib().qmm_gguf_find(self.h, name.encode())

    def tensors(self):
        return [self.info(i) for i in range(len(self))]

    def read(self, name_or_index):
        """The tensor's raw bytes as a numpy uint8 array (host)."""
        i = name_or_index if isinstance(name_or_index, int) else self.find(name_or_index)
        if i < 0:
            raise KeyError(name_or_index)
        out = np.empty(self.info(i)["bytes"], dtype=np.uint8)
        check(lib().qmm_gguf_read_tensor(self.h, i, out.ctypes.data_as(C.c_void_p), out.size), "qmm_gguf_read_tensor")
        return out

    def upload(self, name_or_index, device_tensor):
        """The tensor's raw bytes into a torch CUDA uint8 tensor (pinned bounce buffer, 64 MiB chunks)."""
        import torch
        i = name_or_index if isinstance(name_or_index, int) else self.find(name_or_index)
        if i < 0:
            raise KeyError(name_or_index)
        check(lib().qmm_gguf_upload_tensor(self.h, i, device_tensor.data_ptr(), device_tensor.numel() * device_tensor.element_size(),
                                           torch.cuda.current_stream().cuda_stream), "qmm_gguf_upload_tensor")

    def meta_int(self, key):
        v = C.c_ulonglong()
        check(lib().qmm_gguf_meta_u64(self.h, key.encode(), C.byref(v)), f"qmm_gguf_meta_u64({key})")
        return v.value

    def meta_float(self, key):
        v = C.c_double()
        check(lib().qmm_gguf_meta_f64(self.h, key.encode(), C.byref(v)), f"qmm_gguf_meta_f64({key})")
        return v.value

    def meta_str(self, key):
        n = lib().qmm_gguf_meta_str(self.h, key.encode(), None, 0)
        if n < 0:
            check(int(n), f"qmm_gguf_meta_str({key})")
        buf = C.create_string_buffer(n + 1)
        lib().qmm_gguf_meta_str(self.h, key.encode(), buf, n + 1)
        return buf.value.decode()


class GgufWriter:
    def __init__(self, path):
        self.h = C.c_void_p()
        check(lib().qmm_gguf_writer_create(str(path).encode(), C.byref(self.h)), "qmm_gguf_writer_create")

    def meta(self, key, value):
        L = lib()
        if isinstance(value, str):
            check(L.qmm_gguf_writer_meta_str(self.h, key.encode(), value.encode()), "qmm_gguf_writer_meta_str")
        elif isinstance(value, float):
            check(L.qmm_gguf_writer_meta_f32(self.h, key.encode(), value), "qmm_gguf_writer_meta_f32")
        else:
            check(L.qmm_gguf_writer_meta_u32(self.h, key.encode(), int(value)), "qmm_gguf_writer_meta_u32")
        return self

    def tensor(self, name, qtype, dims, data):
        """dims = [row length k, rows n, ...]; data: numpy array holding the packed bytes."""
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        d = (C.c_long * len(dims))(*dims)
        check(lib().qmm_gguf_writer_add_tensor(self.h, name.encode(), qtype, len(dims), d, data.ctypes.data_as(C.c_void_p), data.size),
              f"qmm_gguf_writer_add_tensor({name})")
        return self

    def finish(self):
        h, self.h = self.h, None
        check(lib().qmm_gguf_writer_finish(h), "qmm_gguf_writer_finish")
