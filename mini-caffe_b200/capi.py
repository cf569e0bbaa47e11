"""ctypes binding over the mini-caffe C API (include/caffe/c_api.h).

One `CaffeLibrary` object wraps one shared object.  The same class drives the
B200 engine (`libcaffe.so`, built from csrc/) and, in tests and the CPU
baseline leg of the benchmark, the reference project's own CPU build, because
both export the identical 25-function C API (reference: include/caffe/c_api.h:26-162,
python/minicaffe/base.py:40-47).
"""
import ctypes
import os

import numpy as np

_real_p = ctypes.POINTER(ctypes.c_float)
_void_p = ctypes.c_void_p
_int_p = ctypes.POINTER(ctypes.c_int)


class CaffeError(RuntimeError):
    """A C API call returned -1; the message is CaffeGetLastError()."""


class CaffeLibrary(object):
    """Loads a libcaffe-compatible shared object and declares its C entry points."""

    def __init__(self, path):
        if not os.path.isfile(path):
            raise FileNotFoundError(path)
        self.path = os.path.abspath(path)
        # RTLD_LOCAL: two libraries exporting the same C++ symbols (engine and
        # reference build) must not interpose on each other in one process.
        self.lib = ctypes.CDLL(self.path, mode=ctypes.RTLD_LOCAL)
        L = self.lib
        L.CaffeGetLastError.restype = ctypes.c_char_p
        L.CaffeBlobData.restype = _real_p
        for name in ("CaffeBlobNum", "CaffeBlobChannels", "CaffeBlobHeight", "CaffeBlobWidth",
                     "CaffeBlobCount", "CaffeBlobData"):
            getattr(L, name).argtypes = [_void_p]
        L.CaffeBlobReshape.argtypes = [_void_p, ctypes.c_int, _int_p]
        L.CaffeBlobShape.argtypes = [_void_p, _int_p, ctypes.POINTER(_int_p)]
        L.CaffeNetCreate.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.POINTER(_void_p)]
        L.CaffeNetCreateFromBuffer.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_char_p,
                                               ctypes.c_int, ctypes.POINTER(_void_p)]
        L.CaffeNetDestroy.argtypes = [_void_p]
        L.CaffeNetMarkOutput.argtypes = [_void_p, ctypes.c_char_p]
        L.CaffeNetForward.argtypes = [_void_p]
        L.CaffeNetGetBlob.argtypes = [_void_p, ctypes.c_char_p, ctypes.POINTER(_void_p)]
        L.CaffeNetListBlob.argtypes = [_void_p, _int_p, ctypes.POINTER(ctypes.POINTER(ctypes.c_char_p)),
                                       ctypes.POINTER(ctypes.POINTER(_void_p))]
        L.CaffeNetListParam.argtypes = L.CaffeNetListBlob.argtypes
        L.CaffeProfilerScopeStart.argtypes = [ctypes.c_char_p]
        L.CaffeProfilerDump.argtypes = [ctypes.c_char_p]
        L.CaffeSetMode.argtypes = [ctypes.c_int, ctypes.c_int]

    def check(self, ret):
        if ret != 0:
            raise CaffeError(self.lib.CaffeGetLastError().decode("utf-8", "replace"))

    def gpu_available(self):
        return bool(self.lib.CaffeGPUAvailable())

    def set_mode(self, gpu, device):
        self.check(self.lib.CaffeSetMode(1 if gpu else 0, device))

    def memory_pool_clear(self):
        self.check(self.lib.CaffeMemoryPoolClear())

    def has(self, symbol):
        return hasattr(self.lib, symbol)


class Blob(object):
    """Borrowed handle to a caffe::Blob owned by a net."""

    def __init__(self, library, handle):
        self._lib = library
        self.handle = handle

    @property
    def shape(self):
        n = ctypes.c_int()
        dims = _int_p()
        self._lib.check(self._lib.lib.CaffeBlobShape(self.handle, ctypes.byref(n), ctypes.byref(dims)))
        return tuple(dims[i] for i in range(n.value))

    @property
    def count(self):
        return self._lib.lib.CaffeBlobCount(self.handle)

    def reshape(self, *shape):
        arr = (ctypes.c_int * len(shape))(*shape)
        self._lib.check(self._lib.lib.CaffeBlobReshape(self.handle, len(shape), arr))

    @property
    def data(self):
        """numpy view on the blob's host memory (CaffeBlobData marks the host copy as
        the authoritative one, as the reference does: c_api.cpp:33-35)."""
        shape = self.shape
        count = int(np.prod(shape)) if shape else 0
        ptr = self._lib.lib.CaffeBlobData(self.handle)
        if count == 0:
            return np.zeros(shape, dtype=np.float32)
        buf = (ctypes.c_float * count).from_address(ctypes.addressof(ptr.contents))
        return np.frombuffer(buf, dtype=np.float32).reshape(shape)


class Net(object):
    """Owns a NetHandle created from prototxt/caffemodel paths or in-memory buffers."""

    def __init__(self, library, prototxt, caffemodel=None, from_buffer=False):
        self._lib = library
        self.handle = _void_p()
        if from_buffer:
            pb = prototxt if isinstance(prototxt, bytes) else prototxt.encode()
            mb = caffemodel or b""
            library.check(library.lib.CaffeNetCreateFromBuffer(pb, len(pb), mb, len(mb),
                                                               ctypes.byref(self.handle)))
        else:
            library.check(library.lib.CaffeNetCreate(prototxt.encode(), (caffemodel or "").encode(),
                                                     ctypes.byref(self.handle)))

    def close(self):
        if self.handle:
            self._lib.lib.CaffeNetDestroy(self.handle)
            self.handle = _void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:  # interpreter shutdown
            pass

    def blob(self, name):
        h = _void_p()
        self._lib.check(self._lib.lib.CaffeNetGetBlob(self.handle, name.encode(), ctypes.byref(h)))
        return Blob(self._lib, h)

    def _list(self, fn):
        n = ctypes.c_int()
        names = ctypes.POINTER(ctypes.c_char_p)()
        handles = ctypes.POINTER(_void_p)()
        self._lib.check(fn(self.handle, ctypes.byref(n), ctypes.byref(names), ctypes.byref(handles)))
        return [(names[i].decode(), Blob(self._lib, _void_p(handles[i]))) for i in range(n.value)]

    def blobs(self):
        return self._list(self._lib.lib.CaffeNetListBlob)

    def params(self):
        """[(display name, Blob)] in net order; display name is '<layer>_<index>' unless the
        prototxt names the param (reference: net.cpp:128-145)."""
        return self._list(self._lib.lib.CaffeNetListParam)

    def mark_output(self, name):
        self._lib.check(self._lib.lib.CaffeNetMarkOutput(self.handle, name.encode()))

    def forward(self, **inputs):
        for k, v in inputs.items():
            b = self.blob(k)
            b.reshape(*v.shape)
            b.data[...] = v
        self._lib.check(self._lib.lib.CaffeNetForward(self.handle))

    def set_params(self, weights):
        """weights: {display name: ndarray}; every listed param must exist and match in size."""
        have = dict(self.params())
        for name, arr in weights.items():
            if name not in have:
                raise KeyError("net has no param named %r" % name)
            dst = have[name].data
            if dst.size != arr.size:
                raise ValueError("param %s: size %d != %d" % (name, dst.size, arr.size))
            dst[...] = np.asarray(arr, dtype=np.float32).reshape(dst.shape)
