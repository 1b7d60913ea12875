"""ctypes binding of include/poplibs_b200.h (one-to-one, no logic of its own)."""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libpoplibs_b200.so")

HALF, FLOAT, QUARTER, BFLOAT16 = 0, 1, 2, 3
F143, F152 = 0, 1   # plb_quarter_format
PASS_NONE, PASS_NONE_MATMUL, PASS_INFERENCE_FWD, PASS_TRAINING_FWD, PASS_TRAINING_BWD, \
    PASS_TRAINING_WU, PASS_FC_INFERENCE_FWD, PASS_FC_TRAINING_FWD, PASS_FC_TRAINING_BWD, \
    PASS_FC_TRAINING_WU = range(10)
MAX_DIMS = 3
PLAN_FORCE_RESIDENT_WEIGHTS, PLAN_NO_RESIDENT_WEIGHTS, PLAN_NO_HALO, PLAN_NO_CTA_PAIR, PLAN_FORCE_CTA_PAIR = 1, 2, 4, 8, 16
PLAN_NO_TMA_STORE, PLAN_NO_PDL, PLAN_NO_A_COLLECTOR, PLAN_NO_DUAL_ISSUE = 32, 64, 128, 256
_U3 = C.c_uint32 * MAX_DIMS


class PlbError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[plb status {code}] {message}")
        self.code = code
        self.message = message


class MatmulDesc(C.Structure):
    _fields_ = [("groups", C.c_uint32), ("m", C.c_uint32), ("k", C.c_uint32), ("n", C.c_uint32),
                ("input_type", C.c_int32), ("output_type", C.c_int32), ("partials_type", C.c_int32),
                ("transpose_a", C.c_int32), ("transpose_b", C.c_int32),
                ("alpha", C.c_float), ("beta", C.c_float),
                ("scale_a", C.c_int32), ("scale_b", C.c_int32),
                ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64),
                ("format_a", C.c_int32), ("format_b", C.c_int32)]

    @staticmethod
    def make(m, k, n, groups=1, input_type=HALF, output_type=HALF, transpose_a=False,
             transpose_b=False, alpha=1.0, beta=0.0, scale_a=0, scale_b=0, partials_type=FLOAT,
             format_a=0, format_b=0):
        d = MatmulDesc()
        d.groups, d.m, d.k, d.n = groups, m, k, n
        d.input_type, d.output_type, d.partials_type = input_type, output_type, partials_type
        d.transpose_a, d.transpose_b = int(transpose_a), int(transpose_b)
        d.alpha, d.beta = alpha, beta
        d.scale_a, d.scale_b = scale_a, scale_b
        d.format_a, d.format_b = format_a, format_b
        return d


class ConvParams(C.Structure):
    _fields_ = [("input_type", C.c_int32), ("output_type", C.c_int32),
                ("num_field_dims", C.c_uint32), ("batch", C.c_uint32), ("groups", C.c_uint32),
                ("in_chans_per_group", C.c_uint32), ("out_chans_per_group", C.c_uint32),
                ("field", _U3), ("kernel", _U3),
                ("in_trunc_lo", _U3), ("in_trunc_hi", _U3), ("in_dilation", _U3),
                ("in_pad_lo", _U3), ("in_pad_hi", _U3), ("in_flip", _U3),
                ("k_trunc_lo", _U3), ("k_trunc_hi", _U3), ("k_dilation", _U3),
                ("k_pad_lo", _U3), ("k_pad_hi", _U3), ("k_flip", _U3),
                ("out_trunc_lo", _U3), ("out_trunc_hi", _U3), ("stride", _U3),
                ("out_pad_lo", _U3), ("out_pad_hi", _U3)]

    _VECS = ("in_trunc_lo", "in_trunc_hi", "in_dilation", "in_pad_lo", "in_pad_hi", "in_flip",
             "k_trunc_lo", "k_trunc_hi", "k_dilation", "k_pad_lo", "k_pad_hi", "k_flip",
             "out_trunc_lo", "out_trunc_hi", "stride", "out_pad_lo", "out_pad_hi")

    @staticmethod
    def make(batch, field: Sequence[int], kernel: Sequence[int], in_chans, out_chans, groups=1,
             input_type=HALF, output_type=HALF, **transforms):
        """``transforms`` are per-dimension lists named like the struct fields
        (in_pad_lo, stride, k_dilation, ...); scalars are broadcast."""
        p = ConvParams()
        nd = len(field)
        p.input_type, p.output_type = input_type, output_type
        p.num_field_dims, p.batch, p.groups = nd, batch, groups
        p.in_chans_per_group, p.out_chans_per_group = in_chans, out_chans
        for i in range(nd):
            p.field[i], p.kernel[i] = field[i], kernel[i]
            p.in_dilation[i] = p.k_dilation[i] = p.stride[i] = 1
        for name, val in transforms.items():
            if name == "padding":
                names = ("in_pad_lo", "in_pad_hi")
            elif name in ConvParams._VECS:
                names = (name,)
            else:
                raise TypeError(f"unknown ConvParams field {name}")
            if val is None:
                continue
            vals = [int(val)] * nd if isinstance(val, (int, bool)) else [int(v) for v in val]
            for nm in names:
                arr = getattr(p, nm)
                for i in range(nd):
                    arr[i] = vals[i]
        return p

    def output_field(self):
        out = _U3()
        _check(lib().plb_conv_output_field(C.byref(self), out))
        return [int(out[i]) for i in range(self.num_field_dims)]

    def macs(self) -> int:
        return int(lib().plb_conv_macs(C.byref(self)))


class ConvOptions(C.Structure):
    _fields_ = [("pass_", C.c_int32), ("partials_type", C.c_int32), ("tile_n", C.c_int32),
                ("split_k", C.c_int32), ("plan_flags", C.c_int32), ("scale_in", C.c_int32), ("scale_weights", C.c_int32),
                ("format_in", C.c_int32), ("format_weights", C.c_int32), ("reserved", C.c_int32)]

    @staticmethod
    def make(pass_=PASS_NONE, partials_type=FLOAT, tile_n=0, split_k=0, plan_flags=0, scale_in=0,
             scale_weights=0, format_in=0, format_weights=0):
        o = ConvOptions()
        o.pass_, o.partials_type, o.tile_n, o.split_k = pass_, partials_type, tile_n, split_k
        o.plan_flags, o.scale_in, o.scale_weights = plan_flags, scale_in, scale_weights
        o.format_in, o.format_weights = format_in, format_weights
        return o


class Plan(C.Structure):
    _fields_ = [("kernel", C.c_int32), ("tile_m", C.c_int32), ("tile_n", C.c_int32),
                ("tile_k_bytes", C.c_int32), ("box_w", C.c_int32), ("box_h", C.c_int32),
                ("box_n", C.c_int32), ("stages", C.c_int32), ("split_k", C.c_int32),
                ("grid", C.c_int32), ("tiles", C.c_int32), ("b_mn_major", C.c_int32),
                ("resident_weights", C.c_int32), ("halo_rows", C.c_int32), ("cta_pair", C.c_int32),
                ("reserved", C.c_int32), ("flops", C.c_uint64), ("bytes", C.c_uint64), ("workspace_bytes", C.c_uint64)]

    def as_dict(self):
        return {n: int(getattr(self, n)) for n, _ in self._fields_}


_LIB = None

# every symbol include/poplibs_b200.h declares
SYMBOLS = (
    "plb_last_error", "plb_version", "plb_context_create", "plb_context_create_on_stream",
    "plb_context_destroy", "plb_context_stream", "plb_synchronize", "plb_launch_count", "plb_device_pci_address",
    "plb_malloc", "plb_free", "plb_memcpy_h2d", "plb_memcpy_d2h", "plb_memset",
    "plb_matmul", "plb_matmul_host", "plb_conv_validate", "plb_conv_output_field",
    "plb_conv_input_index", "plb_conv_macs", "plb_conv_fwd", "plb_convolution",
    "plb_conv_wu_static_scratch", "plb_conv_bwd", "plb_conv_wu",
    "plb_scaled_add_to", "plb_cast_from_f32", "plb_add_bias", "plb_conv_bias_update", "plb_conv_fwd_host",
    "plb_context_set_plan_flags", "plb_norm_moments", "plb_norm_inv_std_dev", "plb_norm_whiten",
    "plb_norm_statistics", "plb_norm_normalise",
    "plb_norm_scale_shift", "plb_norm_param_gradients", "plb_norm_statistics_gradients", "plb_allreduce_f32_p2p", "plb_allreduce_f32_p2p_rs", "plb_conv_wu_allreduce", "plb_conv_wu_allreduce_owners",
    "plb_conv_wu_allreduce_flag_bytes", "plb_allreduce_p2p_signal_bytes", "plb_matmul_host_async",
    "plb_conv_fwd_host_async",
    "plb_rearrange_acts_to_device", "plb_rearrange_acts_from_device",
    "plb_rearrange_weights_to_device", "plb_rearrange_weights_from_device",
    "plb_weights_transpose_chans_flip_xy", "plb_transpose_matrix", "plb_matmul_plan",
    "plb_conv_plan", "plb_conv_wu_plan", "plb_copy_strided", "plb_fill", "plb_timer_start", "plb_timer_stop", "plb_memory_mix_probe",
)


def lib():
    """Loads libpoplibs_b200.so; raises if it is missing (there is no fallback)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(_LIB_PATH):
        raise ImportError(
            f"{_LIB_PATH} is missing: build it with `python -m poplibs_b200.build` "
            "(needs nvcc); poplibs_b200 has no CPU fallback")
    L = C.CDLL(_LIB_PATH)
    vp, u32, u64, i32, sz, f32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int32, C.c_size_t, C.c_float
    CP, MP, OP, PP = C.POINTER(ConvParams), C.POINTER(MatmulDesc), C.POINTER(ConvOptions), C.POINTER(Plan)
    L.plb_last_error.restype = C.c_char_p
    L.plb_version.restype = C.c_char_p
    L.plb_context_create.argtypes = [C.c_int, C.POINTER(vp)]
    L.plb_context_create_on_stream.argtypes = [C.c_int, vp, C.POINTER(vp)]
    L.plb_device_pci_address.argtypes = [C.c_int, C.c_char_p, sz]
    L.plb_memory_mix_probe.argtypes = [vp, i32, i32, sz, vp, vp]
    L.plb_context_destroy.argtypes = [vp]
    L.plb_context_destroy.restype = None
    L.plb_context_stream.argtypes = [vp]
    L.plb_context_stream.restype = vp
    L.plb_synchronize.argtypes = [vp]
    L.plb_launch_count.argtypes = [vp]
    L.plb_launch_count.restype = u64
    L.plb_malloc.argtypes = [vp, sz, C.POINTER(vp)]
    L.plb_free.argtypes = [vp, vp]
    L.plb_memcpy_h2d.argtypes = [vp, vp, vp, sz]
    L.plb_memcpy_d2h.argtypes = [vp, vp, vp, sz]
    L.plb_memset.argtypes = [vp, vp, C.c_int, sz]
    L.plb_matmul.argtypes = [vp, MP, vp, vp, vp, vp]
    L.plb_matmul_host.argtypes = [vp, MP, vp, vp, vp, vp]
    L.plb_matmul_host_async.argtypes = [vp, MP, vp, vp, vp, vp]
    L.plb_conv_validate.argtypes = [CP]
    L.plb_conv_output_field.argtypes = [CP, _U3]
    L.plb_conv_input_index.argtypes = [CP, u32, u32, u32]
    L.plb_conv_macs.argtypes = [CP]
    L.plb_conv_macs.restype = u64
    L.plb_conv_fwd.argtypes = [vp, CP, OP, vp, vp, vp, vp]
    L.plb_convolution.argtypes = [vp, CP, OP, vp, vp, vp, vp, C.c_int]
    L.plb_conv_bwd.argtypes = [vp, CP, OP, vp, vp, vp]
    L.plb_conv_wu.argtypes = [vp, CP, OP, vp, vp, vp, vp]
    L.plb_conv_wu_static_scratch.argtypes = [C.c_int, vp, CP, OP, vp, vp, vp, vp]
    L.plb_scaled_add_to.argtypes = [vp, i32, vp, vp, f32, sz]
    L.plb_cast_from_f32.argtypes = [vp, i32, vp, vp, sz]
    L.plb_add_bias.argtypes = [vp, i32, vp, vp, u64, u32]
    L.plb_conv_bias_update.argtypes = [vp, i32, vp, u64, u32, i32, vp, f32]
    L.plb_allreduce_f32_p2p.argtypes = [vp, i32, i32, C.POINTER(vp), C.POINTER(vp), u32, sz, vp, vp]
    L.plb_norm_moments.argtypes = [vp, i32, vp, u64, u32, f32, vp, vp, vp]
    L.plb_norm_inv_std_dev.argtypes = [vp, i32, vp, vp, u32, f32, f32, i32, vp]
    L.plb_norm_whiten.argtypes = [vp, i32, vp, vp, vp, u64, u32, vp]
    L.plb_norm_statistics.argtypes = [vp, i32, vp, u64, u32, f32, f32, vp, vp, vp]
    L.plb_norm_normalise.argtypes = [vp, i32, vp, vp, vp, vp, vp, u64, u32, vp, vp]
    L.plb_norm_scale_shift.argtypes = [vp, i32, vp, vp, vp, u64, u32, vp]
    L.plb_norm_param_gradients.argtypes = [vp, i32, vp, vp, u64, u32, f32, vp, vp, vp, vp]
    L.plb_norm_statistics_gradients.argtypes = [vp, i32, vp, vp, vp, vp, vp, u64, u32, vp]
    L.plb_context_set_plan_flags.argtypes = [vp, i32]
    L.plb_context_set_plan_flags.restype = None
    L.plb_allreduce_f32_p2p_rs.argtypes = [vp, i32, i32, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), u32, sz,
                                           vp, vp]
    L.plb_conv_wu_allreduce.argtypes = [vp, CP, OP, vp, vp, i32, i32, C.POINTER(vp), C.POINTER(vp), u32, vp, vp]
    L.plb_conv_wu_allreduce_owners.argtypes = [vp, CP, OP, vp, vp, i32, i32, C.POINTER(vp), C.POINTER(vp),
                                               C.POINTER(vp), u32, vp, vp]
    L.plb_conv_wu_allreduce_flag_bytes.argtypes = [CP]
    L.plb_conv_wu_allreduce_flag_bytes.restype = u64
    L.plb_allreduce_p2p_signal_bytes.argtypes = [i32]
    L.plb_allreduce_p2p_signal_bytes.restype = u32
    L.plb_conv_fwd_host.argtypes = [vp, CP, OP, vp, vp, vp, vp]
    L.plb_conv_fwd_host_async.argtypes = [vp, CP, OP, vp, vp, vp, vp]
    for name in ("plb_rearrange_acts_to_device", "plb_rearrange_acts_from_device"):
        getattr(L, name).argtypes = [vp, u32, u32, u32, u64, vp, vp]
    for name in ("plb_rearrange_weights_to_device", "plb_rearrange_weights_from_device",
                 "plb_weights_transpose_chans_flip_xy"):
        getattr(L, name).argtypes = [vp, u32, u32, u32, u32, u64, vp, vp]
    L.plb_transpose_matrix.argtypes = [vp, u32, u32, u32, u32, vp, vp]
    L.plb_copy_strided.argtypes = [vp, u32, u32, C.POINTER(u64), C.POINTER(C.c_int64),
                                   C.POINTER(C.c_int64), vp, vp]
    L.plb_fill.argtypes = [vp, i32, vp, f32, sz]
    L.plb_timer_start.argtypes = [vp]
    L.plb_timer_stop.argtypes = [vp, C.POINTER(f32)]
    L.plb_matmul_plan.argtypes = [MP, PP]
    L.plb_conv_plan.argtypes = [CP, OP, i32, PP]
    L.plb_conv_wu_plan.argtypes = [CP, OP, PP]
    _LIB = L
    return L


def _check(rc: int):
    if rc != 0:
        raise PlbError(rc, lib().plb_last_error().decode("utf-8", "replace"))


def parse_cpulist(text: str):
    """'0-3,8,10-11' (the kernel's cpulist format) -> {0, 1, 2, 3, 8, 10, 11}."""
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def device_local_cpus(device: int):
    """CPUs on the NUMA node the GPU hangs off (sysfs), limited to those this
    process may run on; empty if the platform does not say."""
    buf = C.create_string_buffer(32)
    _check(lib().plb_device_pci_address(device, buf, 32))
    try:
        with open(f"/sys/bus/pci/devices/{buf.value.decode()}/local_cpulist") as f:
            local = parse_cpulist(f.read())
    except (OSError, ValueError):
        return set()
    return local & os.sched_getaffinity(0)


def bind_host_to_device(device: int):
    """Runs the calling thread (and the threads it starts) on the CPUs next to
    the GPU, so that page-locked buffers allocated afterwards land in the
    memory of that NUMA node and the copies of the *_host entry points do not
    cross the socket interconnect.  Returns the previous affinity (pass it to
    os.sched_setaffinity to undo), or None if nothing was changed."""
    cpus = device_local_cpus(device)
    if not cpus:
        return None
    before = os.sched_getaffinity(0)
    if cpus == before:
        return None
    os.sched_setaffinity(0, cpus)
    return before


def _ptr(x) -> Optional[int]:
    """Device/host address of a torch tensor, numpy array, int or None."""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if hasattr(x, "ctypes"):
        return x.ctypes.data
    raise TypeError(f"cannot take the address of {type(x)}")


class Context:
    """plb_context: one device, one stream."""

    def __init__(self, device: int = 0, stream: Optional[int] = None):
        self._h = C.c_void_p()
        if stream is None:
            _check(lib().plb_context_create(device, C.byref(self._h)))
        else:
            _check(lib().plb_context_create_on_stream(device, C.c_void_p(stream), C.byref(self._h)))

    def close(self):
        if self._h:
            lib().plb_context_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self):
        return self._h

    @property
    def stream(self) -> int:
        return int(lib().plb_context_stream(self._h) or 0)

    def synchronize(self):
        _check(lib().plb_synchronize(self._h))

    def memset(self, dst, value: int, nbytes: int):
        """Fills device memory on the context's stream."""
        _check(lib().plb_memset(self._h, _ptr(dst), value, nbytes))

    def launch_count(self) -> int:
        return int(lib().plb_launch_count(self._h))

    def set_plan_flags(self, flags: int):
        """PLAN_* bits added to every plan made for calls through this context."""
        lib().plb_context_set_plan_flags(self._h, int(flags))

    # ---- hot path ---------------------------------------------------------
    def matmul(self, desc: MatmulDesc, a, b, c, d):
        _check(lib().plb_matmul(self._h, C.byref(desc), _ptr(a), _ptr(b), _ptr(c), _ptr(d)))

    def matmul_host(self, desc: MatmulDesc, a, b, c, d, sync: bool = True):
        """Host buffers in, host buffer out.  sync=False returns after enqueueing
        (page-locked buffers; call synchronize() before reading d)."""
        fn = lib().plb_matmul_host if sync else lib().plb_matmul_host_async
        _check(fn(self._h, C.byref(desc), _ptr(a), _ptr(b), _ptr(c), _ptr(d)))

    def conv_fwd(self, p: ConvParams, x, w, out, bias=None, opt: Optional[ConvOptions] = None):
        _check(lib().plb_conv_fwd(self._h, C.byref(p), C.byref(opt) if opt else None,
                                  _ptr(x), _ptr(w), _ptr(bias), _ptr(out)))

    def conv_fwd_host(self, p: ConvParams, x, w, out, bias=None, opt: Optional[ConvOptions] = None,
                      sync: bool = True):
        """Host buffers in, host buffer out.  sync=False returns after enqueueing
        (page-locked buffers; call synchronize() before reading out)."""
        fn = lib().plb_conv_fwd_host if sync else lib().plb_conv_fwd_host_async
        _check(fn(self._h, C.byref(p), C.byref(opt) if opt else None, _ptr(x), _ptr(w), _ptr(bias),
                  _ptr(out)))

    def convolution(self, p: ConvParams, x, w, out, bias=None, opt: Optional[ConvOptions] = None,
                    transpose_and_flip_weights=False):
        _check(lib().plb_convolution(self._h, C.byref(p), C.byref(opt) if opt else None, _ptr(x),
                                     _ptr(w), _ptr(bias), _ptr(out), int(transpose_and_flip_weights)))

    def conv_bwd(self, p: ConvParams, dy, w, dx, opt: Optional[ConvOptions] = None):
        _check(lib().plb_conv_bwd(self._h, C.byref(p), C.byref(opt) if opt else None,
                                  _ptr(dy), _ptr(w), _ptr(dx)))

    def conv_wu(self, p: ConvParams, x, dy, dw, dw_f32=None, opt: Optional[ConvOptions] = None):
        _check(lib().plb_conv_wu(self._h, C.byref(p), C.byref(opt) if opt else None,
                                 _ptr(x), _ptr(dy), _ptr(dw), _ptr(dw_f32)))

    def scaled_add_to(self, dtype, weights, deltas_f32, scale, count):
        _check(lib().plb_scaled_add_to(self._h, dtype, _ptr(weights), _ptr(deltas_f32), scale, count))

    def conv_bias_update(self, acts_dtype, out_grads, pixels, chans, bias_dtype, biases, scale):
        _check(lib().plb_conv_bias_update(self._h, acts_dtype, _ptr(out_grads), pixels, chans,
                                          bias_dtype, _ptr(biases), scale))

    def allreduce_f32_p2p(self, rank, world, buffer_ptrs, signal_pad_ptrs, epoch, count, out_f32, out_half):
        """buffer_ptrs / signal_pad_ptrs: `world` device addresses (ints)."""
        bufs = (C.c_void_p * world)(*[int(p) for p in buffer_ptrs])
        pads = (C.c_void_p * world)(*[int(p) for p in signal_pad_ptrs])
        _check(lib().plb_allreduce_f32_p2p(self._h, rank, world, bufs, pads, epoch, count,
                                           _ptr(out_f32), _ptr(out_half)))

    def conv_wu_allreduce(self, p: ConvParams, x, dy, rank, world, grad_ptrs, flag_ptrs, epoch, dw,
                          dw_f32=None, opt: Optional[ConvOptions] = None, result_ptrs=None):
        """Weight update of this rank's batch slice with the sum over ranks fused
        into the reduction kernel; grad_ptrs / flag_ptrs: `world` device addresses.
        With result_ptrs (`world` addresses of result buffers) every chunk is
        added by one rank and fetched by the others (plb_conv_wu_allreduce_owners)."""
        grads = (C.c_void_p * world)(*[int(v) for v in grad_ptrs])
        flags = (C.c_void_p * world)(*[int(v) for v in flag_ptrs])
        if result_ptrs is None:
            _check(lib().plb_conv_wu_allreduce(self._h, C.byref(p), C.byref(opt) if opt else None, _ptr(x),
                                               _ptr(dy), rank, world, grads, flags, epoch, _ptr(dw),
                                               _ptr(dw_f32)))
            return
        results = (C.c_void_p * world)(*[int(v) for v in result_ptrs])
        _check(lib().plb_conv_wu_allreduce_owners(self._h, C.byref(p), C.byref(opt) if opt else None,
                                                  _ptr(x), _ptr(dy), rank, world, grads, results, flags,
                                                  epoch, _ptr(dw), _ptr(dw_f32)))

    def allreduce_f32_p2p_rs(self, rank, world, input_ptrs, result_ptrs, signal_pad_ptrs, epoch, count,
                             out_f32, out_half):
        """Reduce-scatter + all-gather form; the three tables hold `world` device addresses (ints)."""
        ins = (C.c_void_p * world)(*[int(p) for p in input_ptrs])
        res = (C.c_void_p * world)(*[int(p) for p in result_ptrs])
        pads = (C.c_void_p * world)(*[int(p) for p in signal_pad_ptrs])
        _check(lib().plb_allreduce_f32_p2p_rs(self._h, rank, world, ins, res, pads, epoch, count,
                                              _ptr(out_f32), _ptr(out_half)))

    # ---- batch normalisation (device layout [pixels][chans]) -------------------
    def norm_moments(self, dtype, acts, pixels, chans, scale, centre, mean, power):
        _check(lib().plb_norm_moments(self._h, dtype, _ptr(acts), pixels, chans, scale, _ptr(centre),
                                      _ptr(mean), _ptr(power)))

    def norm_inv_std_dev(self, dtype, mean, power, chans, eps, scale_var, stable, inv_std):
        _check(lib().plb_norm_inv_std_dev(self._h, dtype, _ptr(mean), _ptr(power), chans, eps, scale_var,
                                          int(stable), _ptr(inv_std)))

    def memory_mix_probe(self, reads, writes, nbytes, src, dst):
        """One streaming pass: `reads` (0/1) read and `writes` (0..4) write streams of nbytes each."""
        _check(lib().plb_memory_mix_probe(self._h, reads, writes, nbytes, _ptr(src), _ptr(dst)))

    def norm_statistics(self, dtype, acts, pixels, chans, eps, scale_var, mean, inv_std, power=None):
        """Mean and 1/sigma per channel in one call (the default estimator)."""
        _check(lib().plb_norm_statistics(self._h, dtype, _ptr(acts), pixels, chans, eps, scale_var, _ptr(mean),
                                         _ptr(inv_std), _ptr(power)))

    def norm_normalise(self, dtype, acts, mean, inv_std, gamma, beta, pixels, chans, whitened, out):
        """Whiten, then scale and shift, in one pass; `whitened` may be None."""
        _check(lib().plb_norm_normalise(self._h, dtype, _ptr(acts), _ptr(mean), _ptr(inv_std), _ptr(gamma),
                                        _ptr(beta), pixels, chans, _ptr(whitened), _ptr(out)))

    def norm_whiten(self, dtype, acts, mean, inv_std, pixels, chans, out):
        _check(lib().plb_norm_whiten(self._h, dtype, _ptr(acts), _ptr(mean), _ptr(inv_std), pixels, chans,
                                     _ptr(out)))

    def norm_scale_shift(self, dtype, acts, scale, shift, pixels, chans, out):
        _check(lib().plb_norm_scale_shift(self._h, dtype, _ptr(acts), _ptr(scale), _ptr(shift), pixels,
                                          chans, _ptr(out)))

    def norm_param_gradients(self, dtype, whitened, grads, pixels, chans, scale, gamma_delta, beta_delta,
                             gamma_delta_f32=None, beta_delta_f32=None):
        _check(lib().plb_norm_param_gradients(self._h, dtype, _ptr(whitened), _ptr(grads), pixels, chans,
                                              scale, _ptr(gamma_delta), _ptr(beta_delta),
                                              _ptr(gamma_delta_f32), _ptr(beta_delta_f32)))

    def norm_statistics_gradients(self, dtype, whitened, grads, inv_std, pixels, chans, out,
                                  var_delta=None, mean_delta=None):
        _check(lib().plb_norm_statistics_gradients(self._h, dtype, _ptr(whitened), _ptr(grads),
                                                   _ptr(inv_std), _ptr(var_delta), _ptr(mean_delta),
                                                   pixels, chans, _ptr(out)))

    def cast_from_f32(self, dtype, dst, src, count):
        _check(lib().plb_cast_from_f32(self._h, dtype, _ptr(dst), _ptr(src), count))

    # ---- layouts ----------------------------------------------------------
    def acts_to_device(self, elem_bytes, batch, chans, field_elems, src, dst):
        _check(lib().plb_rearrange_acts_to_device(self._h, elem_bytes, batch, chans, field_elems,
                                                  _ptr(src), _ptr(dst)))

    def acts_from_device(self, elem_bytes, batch, chans, field_elems, src, dst):
        _check(lib().plb_rearrange_acts_from_device(self._h, elem_bytes, batch, chans, field_elems,
                                                    _ptr(src), _ptr(dst)))

    def weights_to_device(self, elem_bytes, groups, co, ci, kelems, src, dst):
        _check(lib().plb_rearrange_weights_to_device(self._h, elem_bytes, groups, co, ci, kelems,
                                                     _ptr(src), _ptr(dst)))

    def weights_from_device(self, elem_bytes, groups, co, ci, kelems, src, dst):
        _check(lib().plb_rearrange_weights_from_device(self._h, elem_bytes, groups, co, ci, kelems,
                                                       _ptr(src), _ptr(dst)))

    def weights_transpose_chans_flip_xy(self, elem_bytes, groups, co, ci, kelems, src, dst):
        _check(lib().plb_weights_transpose_chans_flip_xy(self._h, elem_bytes, groups, co, ci,
                                                         kelems, _ptr(src), _ptr(dst)))

    def copy_strided(self, elem_bytes, shape, src_strides, dst_strides, src, dst):
        n = len(shape)
        _check(lib().plb_copy_strided(self._h, elem_bytes, n, (C.c_uint64 * n)(*shape),
                                      (C.c_int64 * n)(*src_strides), (C.c_int64 * n)(*dst_strides),
                                      _ptr(src), _ptr(dst)))

    def fill(self, dtype, dst, value, count):
        _check(lib().plb_fill(self._h, dtype, _ptr(dst), value, count))

    def transpose_matrix(self, elem_bytes, groups, rows, cols, src, dst):
        _check(lib().plb_transpose_matrix(self._h, elem_bytes, groups, rows, cols, _ptr(src), _ptr(dst)))


def conv_wu_static_scratch(device: int, stream: int, p: ConvParams, x, dy, dw, dw_f32=None,
                           opt: Optional[ConvOptions] = None):
    """plb_conv_wu_static_scratch: the weight gradient without any device
    allocation by the library (no Context is involved)."""
    _check(lib().plb_conv_wu_static_scratch(device, C.c_void_p(stream), C.byref(p),
                                            C.byref(opt) if opt else None, _ptr(x), _ptr(dy),
                                            _ptr(dw), _ptr(dw_f32)))


def matmul_plan(desc: MatmulDesc) -> Plan:
    plan = Plan()
    _check(lib().plb_matmul_plan(C.byref(desc), C.byref(plan)))
    return plan


def conv_wu_plan(p: ConvParams, opt: Optional[ConvOptions] = None) -> Plan:
    """plb_conv_wu_plan: tiling of the weight-update pass."""
    return conv_plan(p, PASS_TRAINING_WU, opt)


def conv_plan(p: ConvParams, pass_: int = PASS_TRAINING_FWD, opt: Optional[ConvOptions] = None) -> Plan:
    plan = Plan()
    if pass_ == PASS_TRAINING_WU:
        _check(lib().plb_conv_wu_plan(C.byref(p), C.byref(opt) if opt else None, C.byref(plan)))
    else:
        _check(lib().plb_conv_plan(C.byref(p), C.byref(opt) if opt else None, pass_, C.byref(plan)))
    return plan
