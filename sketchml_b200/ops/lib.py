"""ctypes binding of libskml_cuda.so (the sm_100a kernels behind a C ABI).

The library is built in-tree by ``sketchml_b200.build`` (nvcc, ``-gencode
arch=compute_100a,code=sm_100a``). On a machine with a GPU a missing or unloadable
library is an error: there is no PyTorch fallback for the kernels."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import build as _build

MAX_PEERS = 16
GPU_MAX_BINS = 4096

_lib: Optional[C.CDLL] = None

# kernels of this library launched so far by this process (the benchmarks report the count)
LAUNCHES = [0]


def count_launches(n: int) -> None:
    LAUNCHES[0] += n

c_ll, c_ull, c_int, c_f, c_d, c_vp = C.c_longlong, C.c_ulonglong, C.c_int, C.c_float, C.c_double, C.c_void_p


class CompressArgs(C.Structure):
    _fields_ = [
        ("keys", c_vp), ("vals", c_vp), ("meta", c_vp), ("n_max", c_ll), ("dim", c_ll),
        ("bin_num", c_ll), ("group_num", c_ll), ("row_num", c_ll), ("col_ratio", c_d),
        ("seed", c_ull), ("step", c_ull), ("rank", c_ll), ("world", c_ll), ("loss_partials", c_vp),
        ("payload", c_vp), ("slot_capacity", c_ll), ("peer_payload", c_vp * MAX_PEERS),
        ("peer_flag", c_vp * MAX_PEERS), ("workspace", c_vp), ("workspace_bytes", c_ll), ("status", c_vp),
        ("budget_cycles", c_ll), ("given_splits", c_vp), ("n_given", c_ll), ("given_min", c_d),
        ("given_max", c_d), ("fused", c_ll), ("grid", c_ll), ("key_encoder", c_ll), ("cell_bits", c_ll), ("quantile_summary", c_ll),
    ]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("payload", c_vp * MAX_PEERS), ("flag", c_vp * MAX_PEERS), ("world", c_ll), ("slot_capacity", c_ll),
        ("step", c_ull), ("dim", c_ll), ("w", c_vp), ("adam_m", c_vp), ("adam_v", c_vp), ("lr", c_d),
        ("adam_scale", c_d), ("acc", c_vp), ("key_scratch", c_vp), ("key_capacity", c_ll), ("loss_out", c_vp),
        ("out_sum", c_vp), ("workspace", c_vp), ("status", c_vp), ("budget_cycles", c_ll), ("fused", c_ll),
        ("grid", c_ll), ("max_groups", c_ll), ("val_scratch", c_vp), ("table_scratch", c_vp), ("table_capacity", c_ll),
        ("weight_sumsq", c_vp), ("reg_out", c_vp), ("reg_lambda", c_d), ("adam_stride", c_ll),
    ]


class StepArgs(C.Structure):
    _fields_ = [
        ("rowptr", c_vp), ("cols", c_vp), ("vals", c_vp), ("labels", c_vp), ("seg_lo", c_ll * 2), ("seg_cnt", c_ll * 2),
        ("nnz_padded", c_ll), ("avg_nnz", c_d), ("w", c_vp), ("g", c_vp), ("bitmap", c_vp), ("loss_id", c_ll),
        ("inv_batch", c_d), ("hot", c_ll), ("partials", c_vp), ("partials_template", c_vp), ("status", c_vp),
        ("budget_cycles", c_ll), ("lam", c_d), ("block_counts", c_vp), ("meta", c_vp), ("keys", c_vp), ("gvals", c_vp),
        ("dense_vals", c_vp), ("n_max", c_ll), ("dim", c_ll), ("compress", C.POINTER(CompressArgs)),
        ("decode", C.POINTER(DecodeArgs)), ("step", c_ull), ("lr", c_d), ("adam_scale", c_d), ("loss_out", c_vp),
        ("t_colptr", c_vp), ("t_rowidx", c_vp), ("t_vals", c_vp), ("t_ucols", c_vp), ("t_bins", c_vp),
        ("t_long_col", c_vp), ("t_long_e0", c_vp), ("t_long_e1", c_vp), ("t_short", c_ll), ("t_medium", c_ll),
        ("t_long", c_ll), ("t_cols", c_ll), ("t_meta", c_vp), ("coef", c_vp),
        ("l_ucols", c_vp), ("l_meta", c_vp), ("l_ncols", c_ll), ("wc", c_vp), ("gc", c_vp),
        ("grad_done_event", c_vp),
        ("tt_tile_pair_ptr", c_vp), ("tt_pair_ptr", c_vp), ("tt_lrow", c_vp), ("tt_pair_dst", c_vp),
        ("tt_col_pair_ptr", c_vp), ("tt_partial", c_vp), ("tt_tiles", c_ll), ("tt_tile_rows", c_ll), ("tt_rows", c_ll),
    ]


_SIGS = {
    "skml_compress_workspace_bytes": (c_ll, [c_ll, c_ll, c_ll, c_ll, c_d, c_ll]),
    "skml_payload_capacity": (c_ll, [c_ll, c_ll, c_ll, c_ll, c_ll, c_d]),
    "skml_compress_splits_offset": (c_ll, [c_ll, c_ll, c_ll, c_ll, c_d, c_ll]),
    "skml_compress_sparse": (c_int, [C.POINTER(CompressArgs), c_vp]),
    "skml_compress_cluster_size": (c_int, []),
    "skml_compress_dense": (c_int, [C.POINTER(CompressArgs), c_vp]),
    "skml_decode_workspace_bytes": (c_ll, [c_ll, c_ll]),
    "skml_decode_update": (c_int, [C.POINTER(DecodeArgs), c_vp]),
    "skml_glm_grad": (c_int, [c_vp, c_vp, c_vp, c_vp, c_ll, c_ll, c_ll, c_d, c_vp, c_vp, c_vp, c_int, c_f, c_int,
                              c_vp, c_vp, c_ll, c_vp]),
    "skml_glm_validate": (c_int, [c_vp, c_vp, c_vp, c_vp, c_ll, c_ll, c_ll, c_d, c_vp, c_int, c_vp, c_vp, c_vp,
                                  c_ll, c_vp]),
    "skml_compact": (c_int, [c_vp, c_vp, c_vp, c_int, c_f, c_vp, c_vp, c_vp, c_vp, c_vp, c_ll, c_vp, c_vp]),
    "skml_compact_blocks": (c_ll, [c_int]),
    "skml_update_dense": (c_int, [c_vp, c_vp, c_vp, c_vp, c_ll, c_f, c_int, c_f, c_f, c_int, c_int, c_vp]),
    "skml_update_sparse": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_ll, c_f, c_int, c_f, c_f, c_int, c_vp]),
    "skml_scatter_kv": (c_int, [c_vp, c_vp, c_vp, c_vp, c_ll, c_int, c_vp]),
    "skml_weight_norm_scratch_bytes": (c_ll, []),
    "skml_weight_norm": (c_int, [c_vp, c_ll, c_d, c_vp, c_vp, c_vp, c_vp]),
    "skml_colsum_tiled": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_vp, c_vp, c_f,
                                  c_vp, c_vp, c_vp]),
    "skml_update_gathered": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_ll, c_int, c_f, c_int, c_f, c_f, c_int, c_vp]),
    "skml_gen_wstar": (c_int, [c_vp, c_ll, c_d, c_ull, c_vp]),
    "skml_gen_rows": (c_int, [c_vp, c_vp, c_vp, c_ll, c_ll, c_int, c_int, c_d, c_int, c_int, c_f, c_vp, c_ull, c_vp]),
    "skml_glm_coef": (c_int, [c_vp, c_vp, c_vp, c_vp, c_ll, c_ll, c_ll, c_d, c_vp, c_int, c_f, c_vp, c_vp, c_vp, c_ll, c_vp]),
    "skml_colsum": (c_int, [c_vp] * 8 + [c_int] * 4 + [c_vp, c_vp, c_f, c_vp, c_vp]),
    "skml_sm_count": (c_int, []),
    "skml_da_analyze": (c_int, [c_vp, c_ll, c_vp, c_vp, c_vp, c_vp]),
    "skml_da_widths": (c_int, [c_vp, c_ll, c_vp, c_vp, c_vp, c_vp]),
    "skml_da_pack": (c_int, [c_vp, c_ll, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "skml_da_fixed_iv": (c_int, [c_vp, c_ll, c_int, c_vp, c_vp]),
    "skml_da_zero_count": (c_int, [c_vp, c_ll, c_vp, c_vp]),
    "skml_da_zero_pos": (c_int, [c_vp, c_ll, c_vp, c_ll, c_vp, c_vp]),
    "skml_da_extract": (c_int, [c_vp, c_ll, c_vp, c_vp, c_vp, c_vp]),
    "skml_unpack_batch": (c_int, [c_vp, c_int, c_ll, c_vp, c_vp, c_ll, c_vp, c_vp, c_vp, c_vp]),
    "skml_unpack_batch_varnibbles": (c_int, [c_vp, c_vp, c_vp, c_ll, c_vp, c_vp, c_ll, c_vp, c_vp, c_vp, c_vp]),
    "skml_row_prefix": (c_int, [c_vp, c_ll, c_vp, c_vp]),
    "skml_unpack_batch_varbytes": (c_int, [c_vp, c_vp, c_vp, c_ll, c_vp, c_vp, c_ll, c_vp, c_vp, c_vp, c_vp]),
    "skml_fixedpoint_scratch_bytes": (c_ll, []),
    "skml_fixedpoint_code_bytes": (c_ll, [c_ll, c_int]),
    "skml_fixedpoint_pack": (c_int, [c_vp, c_vp, c_ll, c_int, c_ull, c_vp, c_vp, c_vp, c_vp]),
    "skml_zipml_scratch_bytes": (c_ll, [c_ll]),
    "skml_zipml_code_bytes": (c_int, [c_int]),
    "skml_zipml_table_len": (c_int, [c_int]),
    "skml_zipml_pack": (c_int, [c_vp, c_vp, c_ll, c_int, c_vp, c_ll, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "skml_zipml_unpack_scatter": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_ll, c_ll, c_int, c_int, c_vp, c_vp]),
    "skml_fixedpoint_unpack_scatter": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_ll, c_ll, c_int, c_int, c_vp, c_vp]),
    "skml_train_step": (c_int, [C.POINTER(StepArgs), c_vp]),
    "skml_ipc_get_handle": (c_int, [c_vp, c_vp]),
    "skml_ipc_open_handle": (c_int, [c_vp, C.POINTER(c_vp)]),
    "skml_ipc_close": (c_int, [c_vp]),
    "skml_region_alloc": (c_int, [c_ll, c_vp]),
    "skml_region_free": (c_int, [c_vp]),
    "skml_enable_peer_access": (c_int, [c_int]),
}


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = _build.CUDA_SO
        if not path.exists():
            _build.build_cuda()
        try:
            _lib = C.CDLL(str(path))
        except OSError as e:
            raise RuntimeError(f"cannot load {path}: {e}. Build it with `python -m sketchml_b200.build`.") from e
        for name, (res, args) in _SIGS.items():
            fn = getattr(_lib, name)
            fn.restype = res
            fn.argtypes = args
    return _lib


def available() -> bool:
    return torch.cuda.is_available()


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with CUDA error {rc}")


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def budget_cycles(seconds: float) -> int:
    """clock64() ticks for a wait budget; SM clocks stay below 2.1 GHz."""
    return int(max(seconds, 1e-3) * 2.0e9)
