"""Python loader for the CPU oracle (liboracle.so) — TEST INFRASTRUCTURE ONLY.

Imported by tests/, by the smoke check and by the benchmark's CPU-baseline leg.
The product package never imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

from vpux_plugin_b200 import abi

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "liboracle.so")
_REF_LIB = os.path.join(_HERE, "_ref", "libvpux_ref_types.so")


def build(with_reference=None):
    """Compile liboracle.so; also oracle/_ref when the reference tree is reachable."""
    subprocess.run(["make", "-s", "-C", _HERE], check=True)
    # the reference tree: named by the environment, else a checkout called `reference` beside this repository
    ref_root = os.environ.get("VPUX_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    if with_reference is None:
        with_reference = os.path.isdir(os.path.join(ref_root, "src", "vpux_utils"))
    if with_reference:
        subprocess.run(["make", "-s", "-C", _HERE, "ref", f"REF={ref_root}"], check=True)


class OracleError(RuntimeError):
    def __init__(self, status, msg):
        super().__init__(f"[{status}] {msg}")
        self.status = status


class Oracle:
    """Backend with the same method surface as vpux_plugin_b200.lib.Library, computed on the host."""

    def __init__(self, nthreads=1):
        if not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(os.path.join(_HERE, "vfold_oracle.cpp")):
            build(with_reference=False)
        self.lib = C.CDLL(_LIB)
        self.nthreads = int(nthreads)
        L = self.lib
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f32_to_f16.argtypes = [C.c_uint32]
        L.orc_f32_to_f16_clamped.restype = C.c_uint16
        L.orc_f32_to_f16_clamped.argtypes = [C.c_uint32]
        L.orc_f16_to_f32.restype = C.c_uint32
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_bf16.restype = C.c_uint16
        L.orc_f32_to_bf16.argtypes = [C.c_uint32]
        L.orc_bf16_to_f32.restype = C.c_uint32
        L.orc_bf16_to_f32.argtypes = [C.c_uint16]
        for name in ("orc_f32_to_f8e4m3", "orc_f32_to_f8e5m2"):
            getattr(L, name).restype = C.c_uint8
            getattr(L, name).argtypes = [C.c_uint32]
        for name in ("orc_f8e4m3_to_f32", "orc_f8e5m2_to_f32"):
            getattr(L, name).restype = C.c_uint32
            getattr(L, name).argtypes = [C.c_uint8]
        L.orc_calc_scale_zp.argtypes = [C.c_double, C.c_double, C.c_double, C.c_double, C.POINTER(C.c_double),
                                        C.POINTER(C.c_int64)]
        L.orc_fake_quantize.restype = C.c_float
        L.orc_fake_quantize.argtypes = [C.c_float] * 6
        L.orc_quantize_value.restype = C.c_int64
        L.orc_quantize_value.argtypes = [C.c_float, C.c_double, C.c_int64, C.c_int64, C.c_int64]
        L.orc_dequantize_value.restype = C.c_float
        L.orc_dequantize_value.argtypes = [C.c_int64, C.c_double, C.c_int64]
        L.orc_mult_shift.argtypes = [C.c_double, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
        for name in ("orc_infer_type", "orc_fold", "orc_row_stats", "orc_quantize_fold", "orc_nnz_per_oc",
                     "orc_sparsify", "orc_weights_table", "orc_synth_fill"):
            getattr(L, name).restype = C.c_int

    # -- helpers ----------------------------------------------------------------------------------
    @staticmethod
    def _err():
        return C.create_string_buffer(512)

    @staticmethod
    def _check(st, err):
        if st != 0:
            raise OracleError(st, err.value.decode(errors="replace"))

    # -- scalar helpers -----------------------------------------------------------------------------
    def f32_to_f16(self, bits):
        return self.lib.orc_f32_to_f16(int(bits))

    def f32_to_f16_clamped(self, bits):
        return self.lib.orc_f32_to_f16_clamped(int(bits))

    def f16_to_f32(self, bits):
        return self.lib.orc_f16_to_f32(int(bits))

    def f32_to_bf16(self, bits):
        return self.lib.orc_f32_to_bf16(int(bits))

    def f32_to_f8(self, value, e5m2=False):
        """float -> float8_e4m3 / float8_e5m2 bits"""
        bits = int(np.float32(value).view(np.uint32))
        return int(self.lib.orc_f32_to_f8e5m2(bits) if e5m2 else self.lib.orc_f32_to_f8e4m3(bits))

    def f8_to_f32(self, code, e5m2=False):
        bits = self.lib.orc_f8e5m2_to_f32(int(code)) if e5m2 else self.lib.orc_f8e4m3_to_f32(int(code))
        return float(np.uint32(bits).view(np.float32))

    def calc_scale_zp(self, qmin, qmax, rmin, rmax):
        s, z = C.c_double(), C.c_int64()
        st = self.lib.orc_calc_scale_zp(qmin, qmax, rmin, rmax, C.byref(s), C.byref(z))
        if st != 0:
            raise OracleError(st, "calcScaleAndZeroPoint failed")
        return s.value, z.value

    def quantize_value(self, x, scale, zp, qmin, qmax):
        return self.lib.orc_quantize_value(float(x), float(scale), int(zp), int(qmin), int(qmax))

    def dequantize_value(self, q, scale, zp):
        return self.lib.orc_dequantize_value(int(q), float(scale), int(zp))

    def mult_shift(self, rescale):
        w, m, s = C.c_int32(), C.c_int32(), C.c_int32()
        st = self.lib.orc_mult_shift(float(rescale), C.byref(w), C.byref(m), C.byref(s))
        if st != 0:
            raise OracleError(st, "approximate failed")
        return w.value, m.value, s.value

    # -- fold -----------------------------------------------------------------------------------------
    def infer_type(self, base_type, is_splat, transforms, n, params_cap=1 << 16):
        out = abi.TensorType()
        osplat = C.c_int(0)
        sb = np.zeros(params_cap, np.float64)
        zb = np.zeros(params_cap, np.int64)
        nbytes = C.c_uint64(0)
        err = self._err()
        bt = base_type.pod()
        st = self.lib.orc_infer_type(C.byref(bt), int(is_splat), transforms, n, C.byref(out), C.byref(osplat),
                                     sb.ctypes.data_as(C.c_void_p), zb.ctypes.data_as(C.c_void_p),
                                     C.c_int64(params_cap), C.byref(nbytes), err, C.c_size_t(512))
        self._check(st, err)
        return abi.TType.from_pod(out), bool(osplat.value), nbytes.value

    def fold(self, content, transforms, n, dst, dst_bytes, params_cap=1 << 16):
        out = abi.TensorType()
        sb = np.zeros(params_cap, np.float64)
        zb = np.zeros(params_cap, np.int64)
        written = C.c_uint64(0)
        err = self._err()
        st = self.lib.orc_fold(C.byref(content), transforms, n, dst.ctypes.data_as(C.c_void_p),
                               C.c_uint64(dst_bytes), C.byref(written), C.byref(out),
                               sb.ctypes.data_as(C.c_void_p), zb.ctypes.data_as(C.c_void_p), C.c_int64(params_cap),
                               self.nthreads, err, C.c_size_t(512))
        self._check(st, err)
        return written.value, abi.TType.from_pod(out)

    def row_stats(self, content, spec, n_units):
        scales = np.zeros(n_units, np.float64)
        zps = np.zeros(n_units, np.int64)
        rmin = np.zeros(n_units, np.float32)
        rmax = np.zeros(n_units, np.float32)
        err = self._err()
        st = self.lib.orc_row_stats(C.byref(content), C.byref(spec), scales.ctypes.data_as(C.c_void_p),
                                    zps.ctypes.data_as(C.c_void_p), rmin.ctypes.data_as(C.c_void_p),
                                    rmax.ctypes.data_as(C.c_void_p), C.c_int64(n_units), self.nthreads, err,
                                    C.c_size_t(512))
        self._check(st, err)
        return scales, zps, rmin, rmax

    def quantize_fold(self, content, spec, transforms, n, dst, dst_bytes, outs=None):
        written = C.c_uint64(0)
        err = self._err()
        st = self.lib.orc_quantize_fold(C.byref(content), C.byref(spec), transforms, n,
                                        dst.ctypes.data_as(C.c_void_p), C.c_uint64(dst_bytes), C.byref(written),
                                        C.byref(outs) if outs is not None else None, self.nthreads, err,
                                        C.c_size_t(512))
        self._check(st, err)
        return written.value

    def nnz_per_oc(self, content, oc):
        counts = np.zeros(oc, np.int64)
        err = self._err()
        st = self.lib.orc_nnz_per_oc(C.byref(content), counts.ctypes.data_as(C.c_void_p), self.nthreads, err,
                                     C.c_size_t(512))
        self._check(st, err)
        return counts

    def sparsify(self, content, data, mapbuf, counts):
        written = C.c_uint64(0)
        err = self._err()
        st = self.lib.orc_sparsify(C.byref(content),
                                   data.ctypes.data_as(C.c_void_p) if data is not None else None,
                                   C.c_uint64(data.nbytes if data is not None else 0), C.byref(written),
                                   mapbuf.ctypes.data_as(C.c_void_p) if mapbuf is not None else None,
                                   C.c_uint64(mapbuf.nbytes if mapbuf is not None else 0),
                                   counts.ctypes.data_as(C.c_void_p) if counts is not None else None, self.nthreads,
                                   err, C.c_size_t(512))
        self._check(st, err)
        return written.value

    def weights_table(self, desc, oc):
        table = np.zeros(oc * 4, np.int32)
        err = self._err()
        st = self.lib.orc_weights_table(C.byref(desc), table.ctypes.data_as(C.c_void_p), self.nthreads, err,
                                        C.c_size_t(512))
        self._check(st, err)
        return table

    def synth_fill(self, spec, count):
        dt = abi.DTYPE_NUMPY[spec.dtype]
        out = np.zeros(count, dt)
        self.lib.orc_synth_fill(C.byref(spec), out.ctypes.data_as(C.c_void_p), C.c_uint64(count), self.nthreads)
        return out


class ReferenceTypes:
    """The reference's own float16/bfloat16 classes, compiled unmodified (oracle/_ref). None when not built."""

    def __init__(self):
        self.lib = C.CDLL(_REF_LIB)
        self.lib.ref_f32_to_f16_n.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
        self.lib.ref_f32_to_bf16_n.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]

    @staticmethod
    def available():
        return os.path.exists(_REF_LIB)

    def f32_to_f16(self, bits_u32):
        bits = np.ascontiguousarray(bits_u32, np.uint32)
        out = np.zeros(bits.shape, np.uint16)
        self.lib.ref_f32_to_f16_n(bits.ctypes.data, out.ctypes.data, bits.size)
        return out

    def f32_to_bf16(self, bits_u32):
        bits = np.ascontiguousarray(bits_u32, np.uint32)
        out = np.zeros(bits.shape, np.uint16)
        self.lib.ref_f32_to_bf16_n(bits.ctypes.data, out.ctypes.data, bits.size)
        return out
