"""ctypes mirror of include/rad_abi.h, include/rad_planes.h and include/r3d_b200.h.

Only structure layouts and enumerator values live here; they must track the headers. The
plugin itself is C++/CUDA -- this module exists so that Python harnesses (tests, bench) can
build RadArgs the way the engine or the reference's dlopen tools do
(tools/probe_m4_entry.cpp:48-59 of libr3d).
"""
from __future__ import annotations

import ctypes as C

RAD_ABI_VERSION = 26

RAD_OK, RAD_E_INVAL, RAD_E_UNSUPPORTED, RAD_E_SHAPE, RAD_E_STRIDE, RAD_E_DTYPE, RAD_E_DEVICE = range(7)
STATUS_NAMES = ["RAD_OK", "RAD_E_INVAL", "RAD_E_UNSUPPORTED", "RAD_E_SHAPE", "RAD_E_STRIDE",
                "RAD_E_DTYPE", "RAD_E_DEVICE"]

(RAD_F32, RAD_F16, RAD_BF16, RAD_F8E4M3, RAD_F8E5M2, RAD_FP4E2M1, RAD_E8M0, RAD_U8, RAD_I8,
 RAD_I32, RAD_I64, RAD_U4, RAD_U2, RAD_F64) = range(1, 15)

RAD_MAX_RANK = 8
RAD_PK_INT, RAD_PK_F64, RAD_PK_STR = 0, 1, 2
RAD_C_EQ, RAD_C_LE, RAD_C_GE, RAD_C_DIV, RAD_C_IN = range(5)
RAD_DOMAIN_HOST, RAD_DOMAIN_DEVICE = 0, 1
RAD_ENC_STR = 16
RAD_ENC_MAX_PLANES = 4
RAD_PLANE_TILED = 1
RAD_PLANES_MAGIC = 0x534E4C50
RAD_PLANES_ALIGN = 256

R3D_ARM_AUTO, R3D_ARM_EXACT, R3D_ARM_STREAM, R3D_ARM_TILE, R3D_ARM_PACK = 0, 1, 2, 3, 4


class RadTensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("dtype", C.c_uint32), ("rank", C.c_uint32),
                ("shape", C.c_int64 * RAD_MAX_RANK), ("stride", C.c_int64 * RAD_MAX_RANK)]


class RadParam(C.Structure):
    _fields_ = [("key", C.c_char_p), ("kind", C.c_int), ("ival", C.c_longlong),
                ("ihi", C.c_longlong), ("sval", C.c_char_p), ("dval", C.c_double)]


class RadArgs(C.Structure):
    _fields_ = [("t", C.POINTER(RadTensor)), ("n_t", C.c_int), ("p", C.POINTER(RadParam)),
                ("n_p", C.c_int), ("scratch", C.c_void_p), ("scratch_bytes", C.c_int64),
                ("reserved0", C.c_void_p), ("reserved1", C.c_int), ("reserved2", C.c_int)]


class RadPluginInfo(C.Structure):
    _fields_ = [("kind", C.c_int), ("name", C.c_char_p), ("version", C.c_char_p),
                ("description", C.c_char_p), ("targets", C.c_char_p)]


class RadParamSpec(C.Structure):
    _fields_ = [("name", C.c_char_p), ("type", C.c_int), ("need", C.c_int), ("role", C.c_int)]


class RadOperandSpec(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dir", C.c_int), ("optional", C.c_int)]


class RadOpSchema(C.Structure):
    _fields_ = [("op", C.c_char_p), ("params", C.POINTER(RadParamSpec)), ("n_params", C.c_int),
                ("operands", C.POINTER(RadOperandSpec)), ("n_operands", C.c_int),
                ("doc", C.c_char_p)]


class RadConstraint(C.Structure):
    _fields_ = [("key", C.c_char_p), ("op", C.c_int), ("ival", C.c_longlong),
                ("sval", C.c_char_p)]


class RadKernelInfo(C.Structure):
    _fields_ = [("name", C.c_char_p), ("op", C.c_char_p), ("family", C.c_char_p),
                ("summary", C.c_char_p), ("shapes", C.c_char_p), ("dtypes", C.c_char_p),
                ("domain", C.c_int), ("priority", C.c_int),
                ("constraints", C.POINTER(RadConstraint)), ("n_constraints", C.c_int),
                ("tunables", C.c_void_p), ("n_tunables", C.c_int), ("reserved", C.c_void_p),
                ("init", C.c_void_p), ("fini", C.c_void_p), ("launch", C.c_void_p),
                ("scratch", C.c_void_p), ("layout", C.c_void_p), ("relayout", C.c_void_p),
                ("opd_shape", C.c_void_p), ("unrelayout", C.c_void_p),
                ("replaces", C.c_char_p)]


class RadEncPlane(C.Structure):
    _fields_ = [("role", C.c_char * RAD_ENC_STR), ("kind", C.c_int), ("dtype", C.c_uint32),
                ("block", C.c_int64 * 2)]


class RadEncoding(C.Structure):
    _fields_ = [("scheme", C.c_char * RAD_ENC_STR), ("n_planes", C.c_int),
                ("transform", C.c_char * RAD_ENC_STR),
                ("plane", RadEncPlane * RAD_ENC_MAX_PLANES)]


class RadLayout(C.Structure):
    _fields_ = [("bytes", C.c_int64), ("align", C.c_int64), ("tag", C.c_char_p)]


class RadPlanesHeader(C.Structure):
    _fields_ = [("magic", C.c_uint32), ("n_planes", C.c_uint32),
                ("transform", C.c_char * RAD_ENC_STR), ("bytes", C.c_int64)]


class RadPlanesEntry(C.Structure):
    _fields_ = [("role", C.c_char * RAD_ENC_STR), ("dtype", C.c_uint32), ("kind", C.c_int32),
                ("block", C.c_int64 * 2), ("rows", C.c_int64), ("cols", C.c_int64),
                ("row_bytes", C.c_int64), ("offset", C.c_int64)]


class R3dGemmQ(C.Structure):
    _fields_ = [("a", C.c_void_p), ("a_scale", C.c_void_p), ("b", C.c_void_p),
                ("b_scale", C.c_void_p), ("y", C.c_void_p),
                ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
                ("as_cols", C.c_int32), ("bs_cols", C.c_int32), ("rblk", C.c_int32),
                ("bs_dtype", C.c_int32),
                ("a_pitch", C.c_int64), ("b_pitch", C.c_int64), ("y_pitch", C.c_int64),
                ("as_pitch", C.c_int64), ("bs_pitch", C.c_int64),
                ("arm", C.c_int32), ("reserved", C.c_int32)]


class R3dW2A8(C.Structure):
    _fields_ = [("a", C.c_void_p), ("a_scale", C.c_void_p), ("b", C.c_void_p), ("scale", C.c_void_p),
                ("zero", C.c_void_p), ("a_sum", C.c_void_p), ("y", C.c_void_p),
                ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("mpad", C.c_int32),
                ("zero_u4", C.c_int32), ("arm", C.c_int32),
                ("a_pitch", C.c_int64), ("as_pitch", C.c_int64), ("y_pitch", C.c_int64),
                ("b_pitch", C.c_int64), ("zp_pitch", C.c_int64), ("sc_pitch", C.c_int64)]


class R3dLogits(C.Structure):
    _fields_ = [("x", C.c_void_p), ("codes", C.c_void_p), ("scale", C.c_void_p),
                ("y", C.c_void_p),
                ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("br", C.c_int32),
                ("scale_dtype", C.c_int32), ("y_dtype", C.c_int32), ("head_fmt", C.c_int32),
                ("arm", C.c_int32),
                ("x_pitch", C.c_int64), ("code_pitch", C.c_int64), ("y_pitch", C.c_int64),
                ("scale_pitch", C.c_int64)]


def planes_round(x: int) -> int:
    return (x + RAD_PLANES_ALIGN - 1) // RAD_PLANES_ALIGN * RAD_PLANES_ALIGN
