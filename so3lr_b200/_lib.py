"""ctypes binding of libso3lr_b200.so (the C ABI declared in include/so3lr_b200.h).

There is no CPU path: if the shared library is missing the import fails with instructions to build it, and every
compute call fails when no CUDA device is present.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libso3lr_b200.so")

STATUS = {0: "ok", 1: "invalid argument", 2: "CUDA error", 3: "neighbor list overflow", 4: "non-finite positions",
          5: "system too large"}


class So3lrB200Error(RuntimeError):
    def __init__(self, status, where):
        super().__init__(f"so3lr_b200: {where} failed: {STATUS.get(status, status)} (status {status})")
        self.status = status


class Options(C.Structure):
    _fields_ = [("cutoff_lr", C.c_float), ("damping", C.c_float), ("skin", C.c_float), ("lr_both_directions", C.c_int),
                ("lr_list_cutoff", C.c_float)]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found. Build it with `python so3lr_b200/build.py` (needs nvcc); "
            "so3lr_b200 has no CPU fallback.")
    lib = C.CDLL(LIB_PATH)
    p, i32, i64, f32, f64 = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_double
    sig = {
        "so3lr_b200_version": (i32, []),
        "so3lr_b200_status_string": (C.c_char_p, [i32]),
        "so3lr_b200_model_create": (i32, [p, C.c_size_t, i32, C.POINTER(p)]),
        "so3lr_b200_model_destroy": (i32, [p]),
        "so3lr_b200_system_create": (i32, [p, i32, p, i32, p, p, p, p, C.POINTER(Options), C.POINTER(p)]),
        "so3lr_b200_system_destroy": (i32, [p]),
        "so3lr_b200_system_set_cell": (i32, [p, p]),
        "so3lr_b200_system_defer_skin_test": (i32, [p, i32, f32]),
        "so3lr_b200_system_compute": (i32, [p, p, p, p, p, p, p, p, p]),
        "so3lr_b200_system_compute_host": (i32, [p, p, p, p, p, p, p]),
        "so3lr_b200_system_aux": (i32, [p, C.POINTER(p), C.POINTER(p), C.POINTER(p)]),
        "so3lr_b200_system_stats": (i32, [p, C.POINTER(i64), C.POINTER(i64), C.POINTER(i64), C.POINTER(i64)]),
        "so3lr_b200_system_graph_replays": (i32, [p, C.POINTER(i64)]),
        "so3lr_b200_system_valid_edges": (i32, [p, C.POINTER(i64)]),
        "so3lr_b200_pack_rows": (i32, [p, i32, C.POINTER(p), C.POINTER(i32), p, i64, p]),
        "so3lr_b200_unpack_rows": (i32, [p, i32, C.POINTER(p), C.POINTER(i32), p, i64, p]),
        "so3lr_b200_system_export_list": (i32, [p, p, p, i32, p, i64, C.POINTER(i64), C.POINTER(i32)]),
        "so3lr_b200_system_graph_eval": (i32, [p, p, i64, p, p, p, i64, p, p, p, p, p, p, p, p, p]),
        "so3lr_b200_system_set_kspace": (i32, [p, i32, f32, i32, i32, i32]),
        "so3lr_b200_system_graph_eval_kspace": (i32, [p, p, i64, p, p, p, i64, p, p, p, p, p, p, p, p, p, p, p]),
        "so3lr_b200_system_nve": (i32, [p, p, i32, f32, p, p, p, p, p]),
        "so3lr_b200_system_enable_virial": (i32, [p, i32]),
        "so3lr_b200_system_virial": (i32, [p, p, p]),
        "so3lr_b200_nhc_init": (i32, [p, p]),
        "so3lr_b200_nhc_half_steps": (i32, [p, p, i32, i32, i32, f64, f64, f64, f64, i32, i32, p, i32]),
        "so3lr_b200_system_nvt": (i32, [p, p, i32, f32, f64, f64, i32, i32, i32, p, p, p, p, p, p]),
        "so3lr_b200_npt_init": (i32, [p, p]),
        "so3lr_b200_system_npt": (i32, [p, p, i32, f32, f64, f64, f64, f64, i32, i32, i32, p, p, p, p, p, p, p, p]),
        "so3lr_b200_system_rescale_cell": (i32, [p, p]),
        "so3lr_b200_npt_pre": (i32, [p, p, i32, f32, f64, f64, f64, f64, i32, i32, i32, f64, p, p]),
        "so3lr_b200_npt_post": (i32, [p, p, i32, f32, f64, f64, f64, f64, i32, i32, i32, f64, p, p]),
        "so3lr_b200_dd_set_atoms": (i32, [p, i32, p, p, p]),
        "so3lr_b200_dd_begin": (i32, [p, p, p]),
        "so3lr_b200_dd_layer_forward": (i32, [p, p, i32]),
        "so3lr_b200_dd_heads": (i32, [p, p, p, p]),
        "so3lr_b200_dd_pair": (i32, [p, p, p, p, p, p]),
        "so3lr_b200_dd_kspace_cell": (i32, [p, p, f32]),
        "so3lr_b200_dd_kspace_accumulate": (i32, [p, p, p, p, C.POINTER(p), C.POINTER(i64)]),
        "so3lr_b200_dd_kspace_finish": (i32, [p, p, p, p, i32, p]),
        "so3lr_b200_dd_heads_backward": (i32, [p, p, p, i64, p]),
        "so3lr_b200_dd_layer_backward_post": (i32, [p, p, i32]),
        "so3lr_b200_dd_layer_backward_attn": (i32, [p, p, i32]),
        "so3lr_b200_dd_forces": (i32, [p, p, p]),
        "so3lr_b200_dd_buffer": (i32, [p, i32, i32, C.POINTER(p), C.POINTER(i32)]),
        "so3lr_b200_system_profile": (i32, [p, i32]),
        "so3lr_b200_system_profile_read": (i32, [p, i32, p, p, p]),
        "so3lr_b200_neighbor_list_noalloc": (i32, [p, i32, p, p, f32, i32, p, i64, p, p]),
        "so3lr_b200_list_row_total": (i32, [p, p, i32, C.POINTER(i64)]),
        "so3lr_b200_host_sph_harm": (None, [f32, f32, f32, p]),
        "so3lr_b200_host_sph_harm_vjp": (None, [f32, f32, f32, p, p]),
        "so3lr_b200_host_pair_terms": (None, [f32, i32, i32, f32, f32, f32, f32, f32, f32, p]),
        "so3lr_b200_host_kspace_tiles": (i32, [i32, i32, i32, p, C.POINTER(f64)]),
        "so3lr_b200_host_coulomb_chi": (None, [f32, f32, f32, p]),
        "so3lr_b200_host_dispersion_fast": (None, [f32, i32, i32, f32, f32, f32, f32, p]),
        "so3lr_b200_host_zbl": (None, [p, f32, i32, i32, p]),
        "so3lr_b200_host_radial_filter": (None, [p, i32, C.c_double, p, p]),
        "so3lr_b200_host_radial_filter_chebyshev": (None, [p, i32, C.c_double, p, p]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib, sorted(sig)


lib, EXPORTS = _load()


def check(status, where):
    if status != 0:
        raise So3lrB200Error(status, where)
