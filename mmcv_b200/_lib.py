"""ctypes binding of ``libdcn_b200.so`` (the C ABI declared in include/dcn_b200.h).

There is no CPU or PyTorch fallback: if the library is missing, importing the
binding raises, and every entry point fails on a machine without an sm_100a GPU.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, 'lib', 'libdcn_b200.so')

DTYPE_F32, DTYPE_BF16, DTYPE_F16 = 0, 1, 2
MATH_AUTO, MATH_FFMA, MATH_TF32X3, MATH_BF16 = 0, 1, 2, 3
PATH_TCGEN05, PATH_SIMT_TILED, PATH_SIMT_DIRECT = 1, 2, 3
ACT_NONE, ACT_SIGMOID = 0, 1
STATIC_SCRATCH_BYTES = 32 << 20
ABI_VERSION = 6   # DCN_ABI_VERSION of include/dcn_b200.h (DcnFwdParams layout)

# Every symbol include/dcn_b200.h declares.
EXPORTS = ['dcn_abi_version', 'dcn_last_error', 'dcn_fwd_plan',
           'dcn_fwd_workspace_bytes', 'dcn_weight_image_bytes', 'dcn_prepare_weights', 'dcn_fwd', 'dcn_fwd_profiled', 'dcn_fwd_static_scratch',
           'dcn_read_counters', 'dcn_read_status', 'dcn_debug_configure', 'dcn_padded_bytes',
           'dcn_pad_channels_last', 'dcn_conv_workspace_bytes', 'dcn_conv_fwd', 'dcn_to_channels_last', 'dcn_bwd_columns', 'dcn_bwd_input',
           'dcn_bwd_coord',
           'dcn_modulated_deform_conv_forward', 'dcn_deform_conv_forward',
           'dcn_forward_workspace_bytes', 'dcn_msda_forward', 'dcn_msda_backward']


class DcnFwdParams(ctypes.Structure):
    _fields_ = [
        ('input', ctypes.c_void_p), ('offset', ctypes.c_void_p),
        ('mask', ctypes.c_void_p), ('weight', ctypes.c_void_p),
        ('bias', ctypes.c_void_p), ('output', ctypes.c_void_p),
        ('dtype', ctypes.c_int32), ('math_mode', ctypes.c_int32),
        ('N', ctypes.c_int64), ('C', ctypes.c_int64), ('H', ctypes.c_int64),
        ('W', ctypes.c_int64), ('Co', ctypes.c_int64),
        ('kh', ctypes.c_int32), ('kw', ctypes.c_int32),
        ('stride_h', ctypes.c_int32), ('stride_w', ctypes.c_int32),
        ('pad_h', ctypes.c_int32), ('pad_w', ctypes.c_int32),
        ('dil_h', ctypes.c_int32), ('dil_w', ctypes.c_int32),
        ('groups', ctypes.c_int32), ('deform_groups', ctypes.c_int32),
        ('in_stride', ctypes.c_int64 * 4),
        ('offset_batch_stride', ctypes.c_int64),
        ('mask_batch_stride', ctypes.c_int64),
        ('out_batch_stride', ctypes.c_int64),
        ('act', ctypes.c_int32), ('act_lo', ctypes.c_int32),
        ('act_hi', ctypes.c_int32), ('device', ctypes.c_int32),
        ('weight_image', ctypes.c_void_p), ('weight_image_bytes', ctypes.c_int64),
        ('offset_channel_stride', ctypes.c_int64), ('offset_pixel_stride', ctypes.c_int64),
        ('mask_channel_stride', ctypes.c_int64), ('mask_pixel_stride', ctypes.c_int64),
        ('mask_act', ctypes.c_int32), ('reserved0', ctypes.c_int32),
        ('padded_input', ctypes.c_void_p), ('padded_input_bytes', ctypes.c_int64),
    ]


class DcnPlanInfo(ctypes.Structure):
    _fields_ = [
        ('path', ctypes.c_int32), ('launches', ctypes.c_int32),
        ('stages_input', ctypes.c_int32), ('tile_m', ctypes.c_int32),
        ('tile_n', ctypes.c_int32), ('tile_k', ctypes.c_int32),
        ('grid', ctypes.c_int32), ('block', ctypes.c_int32),
        ('smem_bytes', ctypes.c_int64), ('Ho', ctypes.c_int64),
        ('Wo', ctypes.c_int64), ('workspace_bytes', ctypes.c_size_t),
        ('operand_stages', ctypes.c_int32), ('weight_stages', ctypes.c_int32),
        ('producer_layout', ctypes.c_int32), ('kernel_version', ctypes.c_int32),
        ('window_h', ctypes.c_int32), ('window_w', ctypes.c_int32),
        ('table_span', ctypes.c_int32), ('table_slots', ctypes.c_int32),
        ('epilogue_tensor_stores', ctypes.c_int32),
    ]


_lib = None


def load():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f'{LIB_PATH} is missing: build it with `python -m mmcv_b200.build_ext` '
            '(there is no fallback implementation)')
    lib = ctypes.CDLL(LIB_PATH)
    P = ctypes.POINTER
    vp, i32, i64, sz = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_size_t
    lib.dcn_abi_version.restype = ctypes.c_int
    if lib.dcn_abi_version() != ABI_VERSION:
        raise RuntimeError(f'dcn_b200: {LIB_PATH} has ABI version {lib.dcn_abi_version()}, '
                           f'this package needs {ABI_VERSION}; rebuild with mmcv_b200.build_ext')
    lib.dcn_last_error.restype = ctypes.c_char_p
    lib.dcn_fwd_plan.argtypes = [P(DcnFwdParams), P(DcnPlanInfo)]
    lib.dcn_fwd_workspace_bytes.argtypes = [P(DcnFwdParams), P(sz)]
    lib.dcn_fwd.argtypes = [P(DcnFwdParams), vp, sz, vp]
    lib.dcn_weight_image_bytes.argtypes = [P(DcnFwdParams), P(sz)]
    lib.dcn_prepare_weights.argtypes = [P(DcnFwdParams), vp, sz, vp]
    lib.dcn_to_channels_last.argtypes = [vp, vp, i32, i64, i64, i64, i64, P(i64), i32, vp]
    lib.dcn_fwd_profiled.argtypes = [P(DcnFwdParams), vp, sz, vp, P(ctypes.c_float)]
    lib.dcn_fwd_static_scratch.argtypes = [P(DcnFwdParams), vp, P(vp)]
    lib.dcn_bwd_columns.argtypes = [P(DcnFwdParams), i64, i64, vp, vp]
    lib.dcn_bwd_input.argtypes = [P(DcnFwdParams), i64, i64, vp, vp, vp]
    lib.dcn_bwd_coord.argtypes = [P(DcnFwdParams), i64, i64, vp, vp, vp, vp]
    lib.dcn_read_counters.argtypes = [vp, vp, P(ctypes.c_uint64)]
    lib.dcn_read_status.argtypes = [vp, vp, P(i32)]
    lib.dcn_debug_configure.argtypes = [ctypes.c_uint64, i32]
    lib.dcn_padded_bytes.argtypes = [i32, i64, i64, i64, i64, P(sz)]
    lib.dcn_pad_channels_last.argtypes = [vp, vp, i32, i64, i64, i64, i64, P(i64), i32, vp]
    lib.dcn_conv_workspace_bytes.argtypes = [P(DcnFwdParams), P(sz)]
    lib.dcn_conv_fwd.argtypes = [P(DcnFwdParams), vp, sz, vp]
    lib.dcn_modulated_deform_conv_forward.argtypes = (
        [vp] * 6 + [i32] + [i64] * 5 + [i32] * 12 + [vp, sz, vp])
    lib.dcn_deform_conv_forward.argtypes = (
        [vp] * 4 + [i32] + [i64] * 5 + [i32] * 12 + [vp, sz, vp])
    lib.dcn_forward_workspace_bytes.argtypes = (
        [i32, i32] + [i64] * 5 + [i32] * 10 + [P(sz)])
    lib.dcn_msda_forward.argtypes = [vp] * 6 + [i32] + [i64] * 7 + [i32, vp]
    lib.dcn_msda_backward.argtypes = [vp] * 9 + [i32] + [i64] * 7 + [i32, vp]
    for name in EXPORTS:
        getattr(lib, name)  # raises AttributeError if a declared symbol is missing
        if name not in ('dcn_last_error',):
            getattr(lib, name).restype = ctypes.c_int
    _lib = lib
    return lib


def last_error():
    return load().dcn_last_error().decode()


class Unsupported(RuntimeError):
    """DCN_ERR_UNSUPPORTED: a valid problem that this library (or the requested kernel) does
    not take."""


def check(rc):
    if rc == -2:
        raise Unsupported(f'dcn_b200: {last_error()} (code {rc})')
    if rc != 0:
        raise RuntimeError(f'dcn_b200: {last_error()} (code {rc})')
