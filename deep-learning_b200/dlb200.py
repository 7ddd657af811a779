"""ctypes binding of libdlb200.so (the C ABI declared in include/dlb200.h).

``Model`` carries the method names of the reference library's ``DL::v1::Model``
(lib/deep-learning/v1/learner/model.hpp L:752-3384): ``compile``,
``set_layer_activation_function``, ``Set__Layer_Normalization``,
``set_dropout``, ``set_optimizer``, ``forward_pass``, ``compute_error``,
``backward_pass``, ``update_derivatives``, ``update_weights`` ...  Everything
numerical runs in the CUDA library; there is no CPU path, and loading fails
loudly when the library has not been built or no sm_100 GPU is present.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdlb200.so")

_vp, _sz, _i, _f, _d, _cp = C.c_void_p, C.c_size_t, C.c_int, C.c_float, C.c_double, C.c_char_p
_u64 = C.c_uint64


class BrnUnitArrays(C.Structure):
    _fields_ = [(n, _vp) for n in ("mean", "sigma", "mean_average", "sigma_average", "r", "d", "gamma", "beta")]


class DropoutDesc(C.Structure):
    _fields_ = [("type", _i), ("value", _f), ("mask", _vp), ("noise", _vp)]


class OptimizerScalars(C.Structure):
    _fields_ = [(n, _f) for n in ("lr_t", "beta1", "beta2", "epsilon", "lower_bound", "upper_bound", "weight_decay")]


# name -> (restype, argtypes); every symbol include/dlb200.h declares.
SIGNATURES = {
    "dlb_status_string": (_cp, [_i]),
    "dlb_last_error": (_cp, []),
    "dlb_version": (_i, []),
    "dlb_ctx_create": (_i, [C.POINTER(_vp), _i]),
    "dlb_ctx_destroy": (_i, [_vp]),
    "dlb_ctx_sync": (_i, [_vp, C.POINTER(_i)]),
    "dlb_ctx_stream": (_vp, [_vp]),
    "dlb_ctx_set_tensor_core": (_i, [_vp, _i]),
    "dlb_ctx_launch_count": (_u64, [_vp]),
    "dlb_ctx_timer_start": (_i, [_vp]),
    "dlb_ctx_timer_stop": (_i, [_vp, C.POINTER(_f)]),
    "dlb_ctx_gemm_profile": (_i, [_vp, _i]),
    "dlb_ctx_gemm_profile_read": (_i, [_vp, C.POINTER(_u64), C.POINTER(_d), C.POINTER(_d)]),
    "dlb_ctx_comm_profile_read": (_i, [_vp, C.POINTER(_u64), C.POINTER(_d), C.POINTER(_u64), C.POINTER(_d)]),
    "dlb_malloc": (_i, [_vp, C.POINTER(_vp), _sz]),
    "dlb_free": (_i, [_vp, _vp]),
    "dlb_memset": (_i, [_vp, _vp, _i, _sz]),
    "dlb_memcpy_h2d": (_i, [_vp, _vp, _vp, _sz]),
    "dlb_memcpy_d2h": (_i, [_vp, _vp, _vp, _sz]),
    "dlb_memcpy_d2d": (_i, [_vp, _vp, _vp, _sz]),
    "dlb_device_mem_info": (_i, [C.POINTER(_sz), C.POINTER(_sz)]),
    "dlb_host_alloc": (_i, [C.POINTER(_vp), _sz]),
    "dlb_host_free": (_i, [_vp]),
    "dlb_split_tf32": (_i, [_vp, _vp, _vp, _sz]),
    "dlb_split_planes": (_i, [_vp, _vp, _vp, _sz]),
    "dlb_split_planes_2d": (_i, [_vp, _vp, _vp, _i, _i]),
    "dlb_ctx_guard_counters": (_i, [_vp, C.POINTER(_u64), C.POINTER(_u64)]),
    "dlb_ctx_set_guard_strict": (_i, [_vp, _i]),
    "dlb_ctx_guard_resplits": (_i, [_vp, C.POINTER(_u64)]),
    "dlb_ctx_set_gemm_kind": (_i, [_vp, _i]),
    "dlb_ctx_gemm_kind": (_i, [_vp]),
    "dlb_fc_forward": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i]),
    "dlb_fc_backward_input": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i]),
    "dlb_fc_weight_gradient": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i]),
    "dlb_brn_forward_sums": (_i, [_vp, _vp, _i, _i, _vp]),
    "dlb_brn_forward_sums_noalloc": (_i, [_vp, _i, _i, _vp, _vp]),
    "dlb_brn_forward_finalize":(_i, [_vp, _vp, _i, _i, _f, _f, _f, _f, C.POINTER(BrnUnitArrays)]),
    "dlb_fc_forward_activation": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, C.POINTER(DropoutDesc), _vp, _vp, _i, _i, _i]),
    "dlb_fc_backward_input_derivative": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i]),
    "dlb_activation_forward": (_i, [_vp, _vp, C.POINTER(BrnUnitArrays), _i, C.POINTER(DropoutDesc), _vp, _vp, _i, _i]),
    "dlb_softmax_forward": (_i, [_vp, _vp, _vp, _i, _i]),
    "dlb_activation_backward": (_i, [_vp, _vp, _vp, _vp, C.POINTER(BrnUnitArrays), _i, _i, _i, _vp]),
    "dlb_brn_backward_apply": (_i, [_vp, _vp, _vp, _vp, C.POINTER(BrnUnitArrays), _vp, _i, _i, _i]),
    "dlb_brn_backward_param_grads": (_i, [_vp, _vp, _i, _vp, _vp, _i]),
    "dlb_residual_forward": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "dlb_shakedrop_backward": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "dlb_residual_forward_padded": (_i, [_vp, _vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _i]),
    "dlb_shakedrop_backward_window": (_i, [_vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _i, _i]),
    "dlb_model_set_shakedrop_noise": (_i, [_vp, _sz, _vp, _vp, _vp, _sz]),
    "dlb_model_set_uout_noise": (_i, [_vp, _sz, _vp, _sz]),
    "dlb_time_major": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i]),
    "dlb_brn_time_forward_sums": (_i, [_vp, _vp, _i, _i, _i, _vp]),
    "dlb_brn_time_forward_finalize": (_i, [_vp, _vp, _i, _i, _i, _f, _f, _f, _f, C.POINTER(BrnUnitArrays)]),
    "dlb_indrnn_forward": (_i, [_vp, _vp, C.POINTER(BrnUnitArrays), _vp, _i, _vp, _vp, _i, _i, _i]),
    "dlb_indrnn_forward_dropout": (_i, [_vp, _vp, C.POINTER(BrnUnitArrays), _vp, _i, _vp, _f, _vp, _vp, _i, _i, _i]),
    "dlb_indrnn_forward_uout": (_i, [_vp, _vp, C.POINTER(BrnUnitArrays), _vp, _i, _vp, _vp, _vp, _i, _i, _i]),
    "dlb_indrnn_backward_walk": (_i, [_vp, _vp, _vp, _vp, C.POINTER(BrnUnitArrays), _vp, _i, _i, _i, _i]),
    "dlb_indrnn_backward_sums": (_i, [_vp, _vp, _vp, _vp, C.POINTER(BrnUnitArrays), _i, _i, _i, _i, _vp]),
    "dlb_time_fold": (_i, [_vp, _vp, _i, _i, _vp]),
    "dlb_brn_time_backward_apply": (_i, [_vp, _vp, _vp, _vp, C.POINTER(BrnUnitArrays), _vp, _i, _i, _i, _i]),
    "dlb_indrnn_clamp": (_i, [_vp, _vp, _i, _f, _f]),
    "dlb_loss_delta":(_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "dlb_optimizer_step": (_i, [_vp, _i, C.POINTER(OptimizerScalars), _vp, _vp, _vp, _vp, _vp, _vp, _sz]),
    "dlb_clip_gradient": (_i, [_vp, _vp, _sz, _f]),
    "dlb_optimizer_prepare": (_i, [_i, C.POINTER(_f), C.POINTER(_f), C.POINTER(_f), C.POINTER(OptimizerScalars)]),
    "dlb_comm_unique_id": (_i, [C.c_char * 128]),
    "dlb_comm_init": (_i, [_vp, C.c_char * 128, _i, _i]),
    "dlb_comm_world": (_i, [_vp]),
    "dlb_comm_rank": (_i, [_vp]),
    "dlb_allreduce_f32": (_i, [_vp, _vp, _sz]),
    "dlb_allreduce_f64": (_i, [_vp, _vp, _sz]),
    "dlb_allreduce_f32_overlapped": (_i, [_vp, _vp, _sz]),
    "dlb_comm_join": (_i, [_vp]),
    "dlb_comm_peer_exchange": (_i, [_vp]),
    "dlb_peer_exchange_emulated": (_i, [_vp, _i, _sz, _i, _vp, _vp, _i, C.c_uint]),
    "dlb_model_create": (_i, [C.POINTER(_vp), _vp]),
    "dlb_model_destroy": (_i, [_vp]),
    "dlb_model_compile": (_i, [_vp, _sz, _sz, _i, _vp, _vp]),
    "dlb_model_compile2": (_i, [_vp, _sz, _sz, _i, _vp, _vp, _vp]),
    "dlb_gather_rows": (_i, [_vp, _vp, _vp, _vp, _sz, _i]),
    "dlb_scatter_add_rows": (_i, [_vp, _vp, _vp, _vp, _sz, _i]),
    "dlb_lstm_forward_step": (_i, [_vp] * 13 + [_i, _i, _i]),
    "dlb_lstm_backward_step": (_i, [_vp] * 14 + [_i, _i, _i]),
    "dlb_lstm_peephole_gradient": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i]),
    "dlb_model_set_layer_activation_function": (_i, [_vp, _sz, _i]),
    "dlb_model_set_layer_normalization": (_i, [_vp, _sz, _i]),
    "dlb_model_set_dropout": (_i, [_vp, _sz, _i, _f, _i]),
    "dlb_model_set_normalization_momentum_average": (_i, [_vp, _f]),
    "dlb_model_set_normalization_epsilon": (_i, [_vp, _f]),
    "dlb_model_set_brn_r_correction_maximum": (_i, [_vp, _f]),
    "dlb_model_set_brn_d_correction_maximum": (_i, [_vp, _f]),
    "dlb_model_set_loss_fn": (_i, [_vp, _i]),
    "dlb_model_set_optimizer": (_i, [_vp, _i]),
    "dlb_model_set_hparam": (_i, [_vp, _cp, _d]),
    "dlb_model_get_hparam": (_d, [_vp, _cp]),
    "dlb_model_set_weight_decay": (_i, [_vp, _f]),
    "dlb_model_set_l2": (_i, [_vp, _f]),
    "dlb_model_set_max_batch_size": (_i, [_vp, _sz]),
    "dlb_model_set_seq_w": (_i, [_vp, _sz]),
    "dlb_model_seed_weights": (_i, [_vp, C.c_uint]),
    "dlb_model_initialize_weights_with_glorot_uniform": (_i, [_vp]),
    "dlb_model_get_size": (_sz, [_vp, _cp]),
    "dlb_model_layer_info": (_i, [_vp, _sz, _vp]),
    "dlb_model_get_array": (_i, [_vp, _cp, _vp, _sz]),
    "dlb_model_set_array": (_i, [_vp, _cp, _vp, _sz]),
    "dlb_model_get_layer_norm": (_i, [_vp, _sz, _cp, _vp, _sz]),
    "dlb_model_set_layer_norm": (_i, [_vp, _sz, _cp, _vp, _sz]),
    "dlb_model_set_dropout_mask": (_i, [_vp, _sz, _vp, _sz]),
    "dlb_model_set_global_batch": (_i, [_vp, _sz]),
    "dlb_model_set_training_size": (_i, [_vp, _sz]),
    "dlb_model_forward_pass": (_i, [_vp, _sz, _vp]),
    "dlb_model_compute_error": (_i, [_vp, _sz, _vp]),
    "dlb_model_backward_pass": (_i, [_vp, _sz]),
    "dlb_model_update_derivatives": (_i, [_vp, _sz]),
    "dlb_model_merge_derivatives": (_i, [_vp]),
    "dlb_model_update_weights": (_i, [_vp, _sz, _sz]),
    "dlb_model_get_loss": (_i, [_vp, C.POINTER(_d)]),
    "dlb_model_set_propagation": (_i, [_vp, _i]),
    "dlb_model_set_accu_fn": (_i, [_vp, _i]),
    "dlb_model_set_accu_var": (_i, [_vp, _f]),
    "dlb_model_compute_loss": (_i, [_vp, _sz, _vp]),
    "dlb_model_compute_loss_device": (_i, [_vp, _sz, _vp]),
    "dlb_model_get_accuracy": (_i, [_vp, C.POINTER(_d)]),
    "dlb_loss_eval": (_i, [_vp, _i, _i, _f, _vp, _vp, _i, _i, _vp, _vp]),
    "dlb_model_reset_loss": (_i, [_vp]),
    "dlb_model_forward_pass_device": (_i, [_vp, _sz, _vp]),
    "dlb_model_compute_error_device": (_i, [_vp, _sz, _vp]),
    "dlb_model_train_step": (_i, [_vp, _sz, _vp, _vp, C.POINTER(_d)]),
    "dlb_model_train_step_device": (_i, [_vp, _sz, _vp, _vp]),
    "dlb_model_set_clip_gradient": (_i, [_vp, _i, _f]),
    "dlb_minibatch_create": (_i, [C.POINTER(_vp), _vp, _vp, _vp, _sz, _i, _sz, _sz, C.c_uint]),
    "dlb_minibatch_destroy": (_i, [_vp]),
    "dlb_minibatch_get_n_batch": (_sz, [_vp]),
    "dlb_minibatch_examples_per_batch": (_sz, [_vp]),
    "dlb_minibatch_examples_last_batch": (_sz, [_vp]),
    "dlb_minibatch_set_shuffle": (_i, [_vp, _i]),
    "dlb_minibatch_shuffle": (_i, [_vp]),
    "dlb_minibatch_get_order": (_i, [_vp, C.POINTER(_sz), _sz]),
    "dlb_minibatch_train": (_i, [_vp, C.POINTER(_d)]),
    "dlb_model_set_constraint_recurrent_weight": (_i, [_vp, _sz, _f, _f]),
    "dlb_model_set_constraint_recurrent_weight_default": (_i, [_vp, _sz]),
    "dlb_model_get_constraint_recurrent_weight": (_i, [_vp, _sz, C.POINTER(_f), C.POINTER(_f)]),
    "dlb_model_save_params": (_i, [_vp, _cp]),
    "dlb_model_save_spec_params": (_i, [_vp, _cp]),
    "dlb_model_load": (_i, [_vp, _cp, _cp]),
    "dlb_checkpointer_create": (_i, [C.POINTER(_vp), _vp, _cp, _i, _i]),
    "dlb_checkpointer_destroy": (_i, [_vp]),
    "dlb_checkpointer_save": (_i, [_vp, _i]),
    "dlb_checkpointer_step": (_i, [_vp, _i, _i, _i, _i, C.POINTER(_i)]),
    "dlb_checkpointer_load": (_i, [_vp, C.POINTER(_i)]),
    "dlb_noise_uniform": (_i, [_vp, _vp, _sz, _f, _f, _u64, C.c_uint32, C.c_uint32, _u64]),
    "dlb_noise_bernoulli": (_i, [_vp, _vp, _sz, _f, _u64, C.c_uint32, C.c_uint32, _u64]),
    "dlb_model_draw_noise": (_i, [_vp, _sz, _u64, C.c_uint32, _sz]),
    "dlb_model_stage_batch": (_i, [_vp, _sz, _vp, _vp]),
    "dlb_model_train_step_staged": (_i, [_vp, C.POINTER(_d)]),
    "dlb_model_set_loss_lag": (_i, [_vp, _i]),
    "dlb_model_set_sharded_update": (_i, [_vp, _i]),
    "dlb_model_set_training_accuracy": (_i, [_vp, _i]),
    "dlb_minibatch_get_accuracy": (_d, [_vp]),
    "dlb_model_get_layer_outputs": (_i, [_vp, _sz, _sz, _vp]),
    "dlb_model_get_layer_errors": (_i, [_vp, _sz, _sz, _i, _vp]),
}

_lib = None


class DlbError(RuntimeError):
    pass


def lib():
    """Loads libdlb200.so; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise DlbError(f"{LIB_PATH} is missing: run `make -C {_HERE}` (there is no CPU fallback)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status, what=""):
    if status != 0:
        L = lib()
        raise DlbError(f"{what}: {L.dlb_status_string(status).decode()} [{L.dlb_last_error().decode()}]")


def _ptr(a):
    return a.ctypes.data_as(_vp)


class Context:
    """One GPU, one stream."""

    def __init__(self, device=0):
        self.L = lib()
        h = _vp()
        check(self.L.dlb_ctx_create(C.byref(h), device), "dlb_ctx_create")
        self.h = h

    def close(self):
        if getattr(self, "h", None):
            self.L.dlb_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def sync(self):
        st = _i(0)
        check(self.L.dlb_ctx_sync(self.h, C.byref(st)), "dlb_ctx_sync")
        return st.value

    def set_tensor_core(self, on):
        check(self.L.dlb_ctx_set_tensor_core(self.h, int(on)), "dlb_ctx_set_tensor_core")

    def set_gemm_kind(self, kind):
        """0: 3xTF32 operands, 1: 3xFP16 planes (the default)."""
        check(self.L.dlb_ctx_set_gemm_kind(self.h, int(kind)), "dlb_ctx_set_gemm_kind")

    def gemm_kind(self):
        return self.L.dlb_ctx_gemm_kind(self.h)

    def guard_counters(self):
        """(operand tensors the range guard flagged, products that ran on the fp32 kernel instead)."""
        a, b = _u64(0), _u64(0)
        check(self.L.dlb_ctx_guard_counters(self.h, C.byref(a), C.byref(b)), "dlb_ctx_guard_counters")
        return int(a.value), int(b.value)

    def guard_resplits(self):
        """Tensors split a second time after outgrowing the scale predicted for them."""
        a = _u64(0)
        check(self.L.dlb_ctx_guard_resplits(self.h, C.byref(a)), "dlb_ctx_guard_resplits")
        return int(a.value)

    def set_guard_strict(self, strict):
        """True: no tensor is exempt from the range guard (call before a model's first batch)."""
        check(self.L.dlb_ctx_set_guard_strict(self.h, int(bool(strict))), "dlb_ctx_set_guard_strict")

    def launch_count(self):
        return int(self.L.dlb_ctx_launch_count(self.h))

    def timer_start(self):
        check(self.L.dlb_ctx_timer_start(self.h), "dlb_ctx_timer_start")

    def timer_stop(self):
        ms = _f(0.0)
        check(self.L.dlb_ctx_timer_stop(self.h, C.byref(ms)), "dlb_ctx_timer_stop")
        return ms.value

    def gemm_profile(self, on):
        check(self.L.dlb_ctx_gemm_profile(self.h, int(on)), "dlb_ctx_gemm_profile")

    def gemm_profile_read(self):
        """(launches, total milliseconds, total algorithmic FLOPs) since the last read."""
        n, ms, fl = _u64(0), _d(0.0), _d(0.0)
        check(self.L.dlb_ctx_gemm_profile_read(self.h, C.byref(n), C.byref(ms), C.byref(fl)), "gemm_profile_read")
        return int(n.value), ms.value, fl.value

    def comm_profile_read(self):
        """(waits for the overlapped all-reduces, their ms, exchanges of sums, their ms) of the
        records the last gemm_profile_read consumed."""
        a, b, c, d = _u64(0), _d(0.0), _u64(0), _d(0.0)
        check(self.L.dlb_ctx_comm_profile_read(self.h, C.byref(a), C.byref(b), C.byref(c), C.byref(d)),
              "comm_profile_read")
        return int(a.value), b.value, int(c.value), d.value

    @property
    def stream(self):
        return self.L.dlb_ctx_stream(self.h)

    # --- device arrays --------------------------------------------------
    def empty(self, shape, dtype=np.float32):
        return DeviceArray(self, shape, dtype)

    def zeros(self, shape, dtype=np.float32):
        a = DeviceArray(self, shape, dtype)
        check(self.L.dlb_memset(self.h, a.ptr, 0, a.nbytes), "dlb_memset")
        return a

    def array(self, host):
        host = np.ascontiguousarray(host)
        a = DeviceArray(self, host.shape, host.dtype)
        a.set(host)
        return a

    # --- communicator ---------------------------------------------------
    def unique_id(self):
        buf = (C.c_char * 128)()
        check(self.L.dlb_comm_unique_id(buf), "dlb_comm_unique_id")
        return bytes(buf)

    def comm_init(self, uid, rank, world):
        buf = (C.c_char * 128).from_buffer_copy(uid)
        check(self.L.dlb_comm_init(self.h, buf, rank, world), "dlb_comm_init")

    def peer_exchange(self):
        """True when the small fp64 sums cross NVLink through peer memory."""
        return bool(self.L.dlb_comm_peer_exchange(self.h))

    def peer_exchange_emulated(self, vectors, rounds=1, absent=-1, wait_ms=20000):
        """The peer-memory exchange with the rows of `vectors` [world, n] as
        emulated ranks on this device; returns what every rank holds after
        `rounds` exchanges (round k on the vectors times k + 1)."""
        v = np.ascontiguousarray(vectors, dtype=np.float64)
        out = np.empty_like(v)
        check(self.L.dlb_peer_exchange_emulated(self.h, v.shape[0], v.shape[1], rounds, _ptr(v), _ptr(out),
                                                absent, wait_ms), "dlb_peer_exchange_emulated")
        return out

    @property
    def world(self):
        return self.L.dlb_comm_world(self.h)

    @property
    def rank(self):
        return self.L.dlb_comm_rank(self.h)


class DeviceArray:
    def __init__(self, ctx, shape, dtype=np.float32):
        self.ctx = ctx
        self.shape = tuple(np.atleast_1d(shape).tolist()) if not isinstance(shape, tuple) else shape
        self.dtype = np.dtype(dtype)
        self.size = int(np.prod(self.shape)) if len(self.shape) else 1
        self.nbytes = self.size * self.dtype.itemsize
        p = _vp()
        check(ctx.L.dlb_malloc(ctx.h, C.byref(p), max(self.nbytes, 16)), "dlb_malloc")
        self.ptr = p

    def set(self, host):
        host = np.ascontiguousarray(host, dtype=self.dtype)
        assert host.size == self.size
        check(self.ctx.L.dlb_memcpy_h2d(self.ctx.h, self.ptr, _ptr(host), self.nbytes), "dlb_memcpy_h2d")
        self.ctx.sync()

    def get(self):
        out = np.empty(self.shape, dtype=self.dtype)
        check(self.ctx.L.dlb_memcpy_d2h(self.ctx.h, _ptr(out), self.ptr, self.nbytes), "dlb_memcpy_d2h")
        return out

    def offset(self, elems):
        return _vp(self.ptr.value + elems * self.dtype.itemsize)

    def free(self):
        if self.ptr is not None and self.ctx.h:
            self.ctx.L.dlb_free(self.ctx.h, self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def device_mem_info():
    """(free, total) bytes of the current CUDA device."""
    free, total = _sz(0), _sz(0)
    check(lib().dlb_device_mem_info(C.byref(free), C.byref(total)), "dlb_device_mem_info")
    return int(free.value), int(total.value)


def pinned_empty(shape, dtype=np.float32):
    """numpy array over page-locked host memory (freed when dropped)."""
    L = lib()
    dtype = np.dtype(dtype)
    n = int(np.prod(shape))
    p = _vp()
    check(L.dlb_host_alloc(C.byref(p), max(n * dtype.itemsize, 16)), "dlb_host_alloc")
    buf = (C.c_char * (n * dtype.itemsize)).from_address(p.value)
    arr = np.frombuffer(buf, dtype=dtype).reshape(shape)
    _PINNED[id(buf)] = (buf, p)
    return arr


_PINNED = {}


class Model:
    backend = "cuda-sm100a"

    def __init__(self, ctx=None, device=0):
        self.L = lib()
        self.ctx = ctx or Context(device)
        h = _vp()
        check(self.L.dlb_model_create(C.byref(h), self.ctx.h), "dlb_model_create")
        self.h = h

    def close(self):
        if getattr(self, "h", None) and self.ctx.h:
            self.L.dlb_model_destroy(self.h)
        self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # --- construction ---------------------------------------------------
    def compile(self, layer_types, layer_units, seq_w=1, model_type=3, allowable_memory=None, layer_units2=None):
        lt = np.ascontiguousarray(layer_types, dtype=np.int32)
        lu = np.ascontiguousarray(layer_units, dtype=np.uint64)
        if layer_units2 is not None:
            lu2 = np.ascontiguousarray(layer_units2, dtype=np.uint64)
            check(self.L.dlb_model_compile2(self.h, len(lt), seq_w, model_type, _ptr(lt), _ptr(lu), _ptr(lu2)), "compile")
            return
        check(self.L.dlb_model_compile(self.h, len(lt), seq_w, model_type, _ptr(lt), _ptr(lu)), "compile")

    def set_layer_activation_function(self, layer, af):
        check(self.L.dlb_model_set_layer_activation_function(self.h, layer, af), "set_layer_activation_function")

    def Set__Layer_Normalization(self, layer, norm):
        check(self.L.dlb_model_set_layer_normalization(self.h, layer, norm), "Set__Layer_Normalization")

    def set_dropout(self, layer, kind, value, scale_weights=False):
        check(self.L.dlb_model_set_dropout(self.h, layer, kind, value, int(scale_weights)), "set_dropout")

    def Set__Normalization_Momentum_Average(self, v):
        check(self.L.dlb_model_set_normalization_momentum_average(self.h, v), "momentum")

    def Set__Normalization_Epsilon(self, v):
        check(self.L.dlb_model_set_normalization_epsilon(self.h, v), "epsilon")

    def Set__Batch_Renormalization_r_Correction_Maximum(self, v):
        check(self.L.dlb_model_set_brn_r_correction_maximum(self.h, v), "r_max")

    def Set__Batch_Renormalization_d_Correction_Maximum(self, v):
        check(self.L.dlb_model_set_brn_d_correction_maximum(self.h, v), "d_max")

    def set_loss_fn(self, loss):
        check(self.L.dlb_model_set_loss_fn(self.h, loss), "set_loss_fn")

    def set_optimizer(self, opt):
        check(self.L.dlb_model_set_optimizer(self.h, opt), "set_optimizer")

    def set_hparam(self, name, value):
        check(self.L.dlb_model_set_hparam(self.h, name.encode(), float(value)), f"set_hparam {name}")

    def get_hparam(self, name):
        return self.L.dlb_model_get_hparam(self.h, name.encode())

    def set_max_batch_size(self, b):
        check(self.L.dlb_model_set_max_batch_size(self.h, b), "set_max_batch_size")

    def set_mp(self, on):
        pass  # OpenMP switch of the reference; the GPU path has nothing to switch

    def set_seq_w(self, delays):
        check(self.L.dlb_model_set_seq_w(self.h, delays), "set_seq_w")

    def set_l2(self, value):
        check(self.L.dlb_model_set_l2(self.h, float(value)), "set_l2")

    def set_weight_decay(self, value):
        check(self.L.dlb_model_set_weight_decay(self.h, float(value)), "set_weight_decay")

    def seed_weights(self, seed):
        check(self.L.dlb_model_seed_weights(self.h, seed), "seed_weights")

    def initialize_weights_with_glorot_uniform(self):
        check(self.L.dlb_model_initialize_weights_with_glorot_uniform(self.h), "glorot")

    def set_global_batch(self, rows):
        check(self.L.dlb_model_set_global_batch(self.h, rows), "set_global_batch")

    def set_training_size(self, n):
        check(self.L.dlb_model_set_training_size(self.h, n), "set_training_size")

    # --- state ----------------------------------------------------------
    def size(self, name):
        v = self.L.dlb_model_get_size(self.h, name.encode())
        if v == 2**64 - 1:
            raise KeyError(name)
        return int(v)

    def layer_info(self, layer):
        out = np.zeros(10, dtype=np.uint64)
        check(self.L.dlb_model_layer_info(self.h, layer, _ptr(out)), "layer_info")
        keys = ("type", "n_out", "first_connection", "last_connection", "first_bias", "last_bias",
                "norm", "dropout", "group", "first_norm_unit")
        return {k: int(v) for k, v in zip(keys, out)}

    def get_array(self, name, n=None):
        n = self.size("total_parameters") if n is None else n
        out = np.empty(n, dtype=np.float32)
        check(self.L.dlb_model_get_array(self.h, name.encode(), _ptr(out), n), f"get_array {name}")
        return out

    def set_array(self, name, arr):
        arr = np.ascontiguousarray(arr, dtype=np.float32)
        check(self.L.dlb_model_set_array(self.h, name.encode(), _ptr(arr), arr.size), f"set_array {name}")

    def get_layer_norm(self, layer, name, n):
        out = np.empty(n, dtype=np.float32)
        check(self.L.dlb_model_get_layer_norm(self.h, layer, name.encode(), _ptr(out), n), f"get_layer_norm {name}")
        return out

    def set_layer_norm(self, layer, name, arr):
        arr = np.ascontiguousarray(arr, dtype=np.float32)
        check(self.L.dlb_model_set_layer_norm(self.h, layer, name.encode(), _ptr(arr), arr.size), f"set_layer_norm {name}")

    def set_dropout_mask(self, layer, mask):
        mask = np.ascontiguousarray(mask, dtype=np.uint8)
        check(self.L.dlb_model_set_dropout_mask(self.h, layer, _ptr(mask), mask.size), "set_dropout_mask")

    def set_shakedrop_noise(self, layer, mask, forward, backward):
        mask = np.ascontiguousarray(mask, dtype=np.uint8)
        forward = np.ascontiguousarray(forward, dtype=np.float32)
        backward = np.ascontiguousarray(backward, dtype=np.float32)
        check(self.L.dlb_model_set_shakedrop_noise(self.h, layer, _ptr(mask), _ptr(forward), _ptr(backward),
                                                   mask.size), "set_shakedrop_noise")

    def set_uout_noise(self, layer, noise):
        noise = np.ascontiguousarray(noise, dtype=np.float32)
        check(self.L.dlb_model_set_uout_noise(self.h, layer, _ptr(noise), noise.shape[0]), "set_uout_noise")

    # --- step -----------------------------------------------------------
    def train_begin(self, batch):
        pass

    @staticmethod
    def _row_pointers(a):
        a = np.ascontiguousarray(a, dtype=np.float32)
        base = a.ctypes.data
        stride = a.strides[0]
        rows = (C.c_void_p * a.shape[0])(*[base + i * stride for i in range(a.shape[0])])
        return a, rows

    def forward_pass(self, batch, X):
        self._x, rows = self._row_pointers(X)
        check(self.L.dlb_model_forward_pass(self.h, batch, rows), "forward_pass")

    def compute_error(self, batch, Y):
        self._y, rows = self._row_pointers(Y)
        check(self.L.dlb_model_compute_error(self.h, batch, rows), "compute_error")

    def set_propagation(self, state):
        check(self.L.dlb_model_set_propagation(self.h, int(state)), "set_propagation")

    def set_accu_fn(self, fn):
        check(self.L.dlb_model_set_accu_fn(self.h, int(fn)), "set_accu_fn")

    def set_accu_var(self, v):
        check(self.L.dlb_model_set_accu_var(self.h, float(v)), "set_accu_var")

    def compute_loss(self, batch, Y):
        self._y, rows = self._row_pointers(Y)
        check(self.L.dlb_model_compute_loss(self.h, batch, rows), "compute_loss")

    def get_accu(self, rows_total=None):
        v = _d(0.0)
        check(self.L.dlb_model_get_accuracy(self.h, C.byref(v)), "get_accuracy")
        return v.value

    def backward_pass(self, batch):
        check(self.L.dlb_model_backward_pass(self.h, batch), "backward_pass")

    def update_derivatives(self, batch):
        check(self.L.dlb_model_update_derivatives(self.h, batch), "update_derivatives")

    def merge_derivatives(self):
        check(self.L.dlb_model_merge_derivatives(self.h), "merge_derivatives")

    def reset_loss(self):
        check(self.L.dlb_model_reset_loss(self.h), "reset_loss")

    def get_loss(self):
        v = _d(0.0)
        check(self.L.dlb_model_get_loss(self.h, C.byref(v)), "get_loss")
        return v.value

    def update_weights(self, batch, training_size):
        check(self.L.dlb_model_update_weights(self.h, batch, training_size), "update_weights")

    def train_step(self, batch, X, Y, want_loss=True):
        X = np.ascontiguousarray(X, dtype=np.float32) if not isinstance(X, np.ndarray) or not X.flags.c_contiguous else X
        Y = np.ascontiguousarray(Y, dtype=np.float32) if not isinstance(Y, np.ndarray) or not Y.flags.c_contiguous else Y
        loss = _d(0.0)
        check(self.L.dlb_model_train_step(self.h, batch, _ptr(X), _ptr(Y), C.byref(loss) if want_loss else None),
              "train_step")
        return loss.value

    def draw_noise(self, batch, seed, step, first_row=0):
        """Draws the next step's dropout masks, UOut and ShakeDrop noise on the device."""
        check(self.L.dlb_model_draw_noise(self.h, batch, seed, step, first_row), "draw_noise")

    def save(self, path_params, path_spec):
        """Model::save_params + Model::save_spec_params."""
        check(self.L.dlb_model_save_params(self.h, path_params.encode()), "save_params")
        check(self.L.dlb_model_save_spec_params(self.h, path_spec.encode()), "save_spec_params")

    def load(self, path_params, path_spec):
        """Model::load into a model that has not been compiled."""
        check(self.L.dlb_model_load(self.h, path_params.encode(), path_spec.encode()), "load")

    def set_clip_gradient(self, use, value):
        check(self.L.dlb_model_set_clip_gradient(self.h, int(bool(use)), float(value)), "set_clip_gradient")

    def set_constraint_recurrent_weight(self, layer, lower, upper):
        check(self.L.dlb_model_set_constraint_recurrent_weight(self.h, layer, float(lower), float(upper)),
              "set_constraint_recurrent_weight")

    def set_constraint_recurrent_weight_default(self, layer):
        check(self.L.dlb_model_set_constraint_recurrent_weight_default(self.h, layer),
              "set_constraint_recurrent_weight_default")

    def get_constraint_recurrent_weight(self, layer):
        lo, hi = _f(0.0), _f(0.0)
        check(self.L.dlb_model_get_constraint_recurrent_weight(self.h, layer, C.byref(lo), C.byref(hi)),
              "get_constraint_recurrent_weight")
        return lo.value, hi.value

    def stage_batch(self, batch, X, Y):
        """Starts the host-to-device copy of one batch; X and Y are contiguous
        float32 arrays (page-locked for an asynchronous copy) that stay
        untouched until the step that uses them has been called."""
        for a in (X, Y):
            if not (isinstance(a, np.ndarray) and a.dtype == np.float32 and a.flags.c_contiguous):
                raise ValueError("stage_batch: contiguous float32 arrays")
        check(self.L.dlb_model_stage_batch(self.h, batch, _ptr(X), _ptr(Y)), "stage_batch")

    def train_step_staged(self, want_loss=True):
        loss = _d(0.0)
        check(self.L.dlb_model_train_step_staged(self.h, C.byref(loss) if want_loss else None),
              "train_step_staged")
        return loss.value

    def set_loss_lag(self, steps):
        """1: train_step_staged returns the loss of the step before (NaN at first)."""
        check(self.L.dlb_model_set_loss_lag(self.h, int(steps)), "set_loss_lag")

    def set_training_accuracy(self, on):
        """True: compute_error keeps the accuracy counter too (get_accuracy after a training pass)."""
        check(self.L.dlb_model_set_training_accuracy(self.h, int(bool(on))), "set_training_accuracy")

    def set_sharded_update(self, on):
        """Several ranks, one-call steps: owner-computes update of the weight matrices
        (default on) or all-reduce and the replicated update."""
        check(self.L.dlb_model_set_sharded_update(self.h, int(bool(on))), "set_sharded_update")

    def train_step_device(self, batch, X_dev, Y_dev):
        check(self.L.dlb_model_train_step_device(self.h, batch, X_dev.ptr, Y_dev.ptr), "train_step_device")

    def get_layer_outputs(self, layer, batch):
        n_out = self.layer_info(layer)["n_out"]
        T = self.size("seq_w")
        out = np.empty((T, batch, n_out), dtype=np.float32)
        check(self.L.dlb_model_get_layer_outputs(self.h, layer, batch, _ptr(out)), "get_layer_outputs")
        return out

    def get_layer_errors(self, layer, batch, which=0):
        n_out = self.layer_info(layer)["n_out"]
        T = self.size("seq_w")
        out = np.empty((T, batch, n_out), dtype=np.float32)
        check(self.L.dlb_model_get_layer_errors(self.h, layer, batch, which, _ptr(out)), "get_layer_errors")
        return out


class MiniBatch:
    """The mini-batch loop of the reference (DL::v1::MiniBatch) over host arrays
    X [n, seq_w * n_in] and Y [n, seq_w * n_out], handed over as row pointers."""

    def __init__(self, model, X, Y, desired_per_batch, use_shuffle=False, max_batches=0, seed=0):
        self.L = model.L
        self.model = model
        self._x, self._xr = Model._row_pointers(X)
        self._y, self._yr = Model._row_pointers(Y)
        self.n = self._x.shape[0]
        self.h = _vp()
        check(self.L.dlb_minibatch_create(C.byref(self.h), model.h, self._xr, self._yr, self.n, int(bool(use_shuffle)),
                                          int(desired_per_batch), int(max_batches), int(seed)), "minibatch_create")

    def close(self):
        if self.h:
            self.L.dlb_minibatch_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def n_batch(self):
        return self.L.dlb_minibatch_get_n_batch(self.h)

    @property
    def per_batch(self):
        return self.L.dlb_minibatch_examples_per_batch(self.h)

    @property
    def last_batch(self):
        return self.L.dlb_minibatch_examples_last_batch(self.h)

    def set_shuffle(self, on):
        check(self.L.dlb_minibatch_set_shuffle(self.h, int(bool(on))), "minibatch_set_shuffle")

    def shuffle(self):
        check(self.L.dlb_minibatch_shuffle(self.h), "minibatch_shuffle")

    def order(self):
        out = (_sz * self.n)()
        check(self.L.dlb_minibatch_get_order(self.h, out, self.n), "minibatch_get_order")
        return np.array(out[:], dtype=np.int64)

    def train(self):
        """One pass over the data set; the mean of the batch losses."""
        v = _d(0.0)
        check(self.L.dlb_minibatch_train(self.h, C.byref(v)), "minibatch_train")
        return v.value

    def accuracy(self):
        """Mean of the batch accuracies of the last pass, in percent."""
        return float(self.L.dlb_minibatch_get_accuracy(self.h))


class Checkpointer:
    """DL::Checkpointer / CheckpointerInterval over a Model: rotating checkpoint
    directories in the reference's layout, plus the optimizer moments."""

    def __init__(self, model, ckpt_dir, max_to_keep=3, interval=1):
        self.L = lib()
        self.model = model
        h = _vp()
        check(self.L.dlb_checkpointer_create(C.byref(h), model.h, os.fsencode(ckpt_dir), max_to_keep, interval),
              "dlb_checkpointer_create")
        self.h = h

    def save(self, step):
        check(self.L.dlb_checkpointer_save(self.h, step), "dlb_checkpointer_save")

    def __call__(self, g, step=None, is_top=True, force=False):
        saved = _i(0)
        check(self.L.dlb_checkpointer_step(self.h, g, g if step is None else step, int(is_top), int(force),
                                           C.byref(saved)), "dlb_checkpointer_step")
        return bool(saved.value)

    def load(self):
        found = _i(0)
        check(self.L.dlb_checkpointer_load(self.h, C.byref(found)), "dlb_checkpointer_load")
        return bool(found.value)

    def __del__(self):
        try:
            if getattr(self, "h", None):
                self.L.dlb_checkpointer_destroy(self.h)
                self.h = None
        except Exception:
            pass
