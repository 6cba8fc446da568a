"""ctypes binding of include/fortis_b200.h."""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


class FortisError(RuntimeError):
    pass


def lib_path():
    """The in-tree library; FORTIS_B200_LIB names another build of it (A/B comparisons)."""
    return os.environ.get("FORTIS_B200_LIB") or os.path.join(HERE, "libfortis_b200.so")


def load():
    """Load libfortis_b200.so (once).  Raises FortisError when it is missing: the CUDA library IS the product and
    nothing else can stand in for it."""
    global _LIB
    if _LIB is not None:
        return _LIB
    p = lib_path()
    if not os.path.exists(p):
        raise FortisError("%s is missing: build it with `python -m fortis_b200.build` (nvcc, sm_100a)" % p)
    L = ctypes.CDLL(p)      # RTLD_LOCAL: the entry names (fortis_gather, mgpuStreamCreate ...) stay out of the global scope
    c = ctypes
    vp, ci, cl, cc = c.c_void_p, c.c_int, c.c_long, c.c_char_p
    sig = {
        "fortis_configure": (ci, [cc, cc]), "fortis_configure_file": (ci, [cc, cc]),
        "fortis_set_vector": (ci, [cc, vp, cl, ci]), "fortis_load_model": (ci, [cc]),
        "fortis_load_model_mem": (ci, [vp, cl]), "fortis_set_option": (ci, [cc, cc]), "fortis_reset": (None, []),
        "fortis_last_error": (ci, []), "fortis_last_error_message": (cc, []), "fortis_sync": (None, []),
        "fortis_gatherv": (None, [c.POINTER(ci), ci, c.POINTER(vp), ci]),
        "fortis_scatterv": (None, [c.POINTER(ci), ci, c.POINTER(vp), ci]),
        "fortis_stepv": (None, [c.POINTER(vp), ci, c.POINTER(vp), ci]),
        "fortis_stepvi": (None, [c.POINTER(ci), ci, c.POINTER(vp), ci, c.POINTER(vp), ci]),
        "mlp_forward_batched": (None, [vp, vp]), "mlp_forward": (None, [vp, vp]), "mlp_upload": (None, [vp]),
        "mlp_forward_dev": (None, []), "mlp_download": (None, [vp]), "fortis_pack": (None, [vp, ci]),
        "fortis_unpack": (None, [vp, ci]), "fortis_model_input": (vp, []), "fortis_model_output": (vp, []),
        "fortis_begin": (None, [ci]), "mgpuStreamCreate": (vp, []), "fortis_alloc": (vp, [cl]), "fortis_free": (None, [vp]),
        "fortis_checksum": (ci, [vp, cl, ci, c.POINTER(c.c_double)]), "fortis_step_checksum": (ci, [c.POINTER(c.c_double)]),
        "fortis_checksum_noalloc": (ci, [vp, cl, ci, vp, vp]),
        "fortis_device_status": (ci, []), "fortis_copy_to_host": (ci, [vp, vp, cl]), "fortis_copy_to_device": (ci, [vp, vp, cl]),
        "fortis_debug_eval_expr": (ci, [cc, ci, c.c_double, c.POINTER(c.c_double), c.POINTER(ci), ci, c.POINTER(c.c_double)]),
        "fortis_debug_plan": (ci, [cc, cc, cc, ci, cl, c.POINTER(ci), ci, c.POINTER(c.c_longlong), c.POINTER(ci),
                                   c.POINTER(ci), ci, c.POINTER(c.c_longlong)]),
    }
    for name, (res, args) in sig.items():
        f = getattr(L, name)
        f.restype = res
        f.argtypes = args
    _LIB = L
    return L


def check(L):
    """Raise if the library recorded an error since the last successful configure."""
    if L.fortis_last_error() != 0:
        raise FortisError(L.fortis_last_error_message().decode())
