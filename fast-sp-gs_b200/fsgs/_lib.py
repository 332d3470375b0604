"""ctypes binding of ``libfsgs.so`` (declarations: ``include/fsgs.h``).

There is no fallback: if the library cannot be loaded every operator raises.
"""
import ctypes
import os
from ctypes import POINTER, Structure, c_float, c_int, c_int32, c_int64, c_size_t, c_uint8, c_void_p

from .build import LIB

_vp = c_void_p


class LBS(Structure):
    _fields_ = [("K", c_int32), ("M", c_int32), ("xyz", _vp), ("scaling_raw", _vp), ("rotation_raw", _vp),
                ("knn_idx", _vp), ("knn_w", _vp), ("sp_q", _vp), ("sp_t", _vp), ("sp_dr", _vp), ("sp_ds", _vp),
                ("sp_pair_offsets", _vp), ("sp_pairs", _vp)]


class LBSGrads(Structure):
    _fields_ = [("g_xyz", _vp), ("g_scaling_raw", _vp), ("g_rotation_raw", _vp), ("g_knn_w", _vp), ("g_sp_q", _vp),
                ("g_sp_t", _vp), ("g_sp_dr", _vp), ("g_sp_ds", _vp), ("accumulate", c_int32), ("scratch_rot", _vp)]


class AdamTensor(Structure):
    _fields_ = [("param", _vp), ("grad", _vp), ("exp_avg", _vp), ("exp_avg_sq", _vp), ("M", c_int32),
                ("lr", c_float), ("eps", c_float)]


class RowTensor(Structure):
    _fields_ = [("src", _vp), ("dst", _vp), ("row_words", c_int32)]


class PreprocessArgs(Structure):
    _fields_ = [("P", c_int32), ("W", c_int32), ("H", c_int32), ("sh_degree", c_int32), ("n_dc", c_int32),
                ("n_rest", c_int32),
                ("means", _vp), ("scales", _vp), ("rots", _vp), ("opac", _vp), ("shs", _vp), ("sh_rest", _vp),
                ("Tw2v", _vp), ("Tv2s", _vp), ("campos", _vp), ("trans_precomp", _vp), ("culling", _vp),
                ("lbs", POINTER(LBS)), ("warped_means", _vp), ("warped_scales", _vp), ("warped_rots", _vp),
                ("means2D", _vp), ("colors", _vp), ("trans_mat", _vp), ("inverse_m", _vp), ("normal_opacity", _vp),
                ("depths", _vp), ("radii", _vp), ("tiles_touched", _vp), ("records", _vp), ("tile_counts", _vp),
                ("counters", _vp), ("opacity_is_logit", c_int32)]


class BinArgs(Structure):
    _fields_ = [("P", c_int32), ("W", c_int32), ("H", c_int32),
                ("means2D", _vp), ("inverse_m", _vp), ("depths", _vp), ("opac", _vp), ("radii", _vp),
                ("tile_counts", _vp), ("counters", _vp), ("capacity", c_int64), ("point_list", _vp), ("ranges", _vp),
                ("tile_order", _vp), ("workspace", _vp), ("workspace_bytes", c_size_t), ("opac_stride", c_int32)]


class RenderArgs(Structure):
    _fields_ = [("P", c_int32), ("W", c_int32), ("H", c_int32), ("near_n", c_float), ("far_n", c_float),
                ("only_image", c_int32), ("records", _vp), ("point_list", _vp), ("ranges", _vp), ("tile_order", _vp),
                ("trans_mat_t2", _vp), ("out_color", _vp), ("out_opacity", _vp), ("out_extras", _vp),
                ("out_flow", _vp), ("n_contrib", _vp), ("accum_max_count", _vp), ("accum_weights_p", _vp),
                ("accum_weights_count", _vp), ("counters", _vp)]


class RenderBwdArgs(Structure):
    _fields_ = [("P", c_int32), ("W", c_int32), ("H", c_int32), ("near_n", c_float), ("far_n", c_float),
                ("records", _vp), ("point_list", _vp), ("ranges", _vp), ("tile_order", _vp), ("trans_mat_t2", _vp),
                ("out_opacity", _vp), ("out_extras", _vp), ("n_contrib", _vp),
                ("dL_dcolor", _vp), ("dL_dopacity", _vp), ("dL_dextras", _vp), ("dL_dflow", _vp),
                ("dL_dcolors", _vp), ("dL_dmeans2D", _vp), ("dL_dtrans_mat", _vp), ("dL_dinverse_m", _vp),
                ("dL_dnormal_opacity", _vp), ("counters", _vp)]


class PreprocessBwdArgs(Structure):
    _fields_ = [("P", c_int32), ("W", c_int32), ("H", c_int32), ("sh_degree", c_int32), ("n_dc", c_int32),
                ("n_rest", c_int32),
                ("means", _vp), ("scales", _vp), ("rots", _vp), ("shs", _vp), ("sh_rest", _vp),
                ("Tw2v", _vp), ("Tv2s", _vp), ("campos", _vp), ("trans_mat", _vp), ("colors", _vp), ("radii", _vp),
                ("grad_means2D", _vp), ("grad_trans_mat", _vp), ("grad_inverse_m", _vp), ("grad_colors", _vp),
                ("grad_normal_opacity", _vp),
                ("grad_means", _vp), ("grad_scales", _vp), ("grad_rots", _vp), ("grad_opac", _vp), ("grad_shs", _vp),
                ("grad_sh_rest", _vp), ("normal_opacity", _vp), ("visible", _vp), ("accumulate", c_int32),
                ("counters", _vp), ("sh_source", _vp)]


class ViewArgs(Structure):
    _fields_ = [("P", c_int32), ("W", c_int32), ("H", c_int32), ("sh_degree", c_int32), ("n_dc", c_int32),
                ("n_rest", c_int32), ("near_n", c_float), ("far_n", c_float),
                ("opacity_raw", _vp), ("sh_dc", _vp), ("sh_rest", _vp), ("lbs", POINTER(LBS)),
                ("Tw2v", _vp), ("Tv2s", _vp), ("campos", _vp),
                ("out_color", _vp), ("out_opacity", _vp), ("out_extras", _vp), ("n_contrib", _vp), ("radii", _vp),
                ("counters", _vp),
                ("dL_dcolor", _vp), ("dL_dopacity", _vp), ("dL_dextras", _vp),
                ("g_xyz", _vp), ("g_scaling_raw", _vp), ("g_rotation_raw", _vp), ("g_opacity_raw", _vp),
                ("g_sh_dc", _vp), ("g_sh_rest", _vp),
                ("g_knn_w", _vp), ("g_sp_q", _vp), ("g_sp_t", _vp), ("g_sp_dr", _vp), ("g_sp_ds", _vp),
                ("visible", _vp), ("viewspace_grad", _vp), ("accumulate", c_int32), ("phase", c_int32),
                ("list_capacity", c_int64), ("workspace", _vp), ("workspace_bytes", c_size_t), ("g_sh_source", _vp)]


class MotionCfg(Structure):
    _fields_ = [("M", c_int32), ("depth", c_int32), ("width", c_int32), ("skip", c_int32), ("deg_p", c_int32),
                ("deg_t", c_int32), ("time_hidden", c_int32), ("time_out", c_int32), ("local_frame", c_int32),
                ("scale_p", c_float), ("scale_t", c_float)]


class MotionArgs(Structure):
    _fields_ = [("cfg", MotionCfg), ("sp_points", _vp), ("t", _vp), ("params", _vp),
                ("sp_q", _vp), ("sp_t", _vp), ("sp_dr", _vp), ("sp_ds", _vp),
                ("g_sp_q", _vp), ("g_sp_t", _vp), ("g_sp_dr", _vp), ("g_sp_ds", _vp), ("g_params", _vp),
                ("accumulate", c_int32), ("workspace", _vp), ("workspace_bytes", c_size_t)]


# every symbol include/fsgs.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "fsgs_status_string": (ctypes.c_char_p, [c_int]),
    "fsgs_version": (c_int, []),
    "fsgs_cdist_top": (c_int, [c_int, c_int, c_int, c_int, _vp, _vp, c_int, _vp, _vp, _vp]),
    "fsgs_cdist_top_backward": (c_int, [c_int, c_int, c_int, c_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "fsgs_cdist_top_f64": (c_int, [c_int, c_int, c_int, c_int, _vp, _vp, c_int, _vp, _vp, _vp]),
    "fsgs_cdist_top_backward_f64": (c_int, [c_int, c_int, c_int, c_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "fsgs_knn": (c_int, [c_int, c_int, c_int, _vp, _vp, _vp, _vp, _vp]),
    "fsgs_knn_grid_workspace_bytes": (c_size_t, [c_int]),
    "fsgs_knn_grid": (c_int, [c_int, c_int, c_int, _vp, _vp, _vp, _vp, _vp, c_size_t, _vp]),
    "fsgs_adam_masked": (c_int, [_vp, _vp, _vp, _vp, _vp, c_float, c_float, c_float, c_float, c_int64, c_int64, _vp]),
    "fsgs_adam_masked_multi": (c_int, [c_int, POINTER(AdamTensor), _vp, c_int64, c_float, c_float, _vp]),
    "fsgs_adam_masked_multi_fmask": (c_int, [c_int, POINTER(AdamTensor), _vp, c_int64, c_float, c_float, _vp]),
    "fsgs_view_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int64, c_int, c_int]),
    "fsgs_motion_param_count": (c_int64, [POINTER(MotionCfg)]),
    "fsgs_motion_param_offsets": (c_int, [POINTER(MotionCfg), POINTER(c_int64), POINTER(c_int32)]),
    "fsgs_motion_workspace_bytes": (c_size_t, [POINTER(MotionCfg)]),
    "fsgs_motion_forward": (c_int, [POINTER(MotionArgs), _vp]),
    "fsgs_motion_backward": (c_int, [POINTER(MotionArgs), _vp]),
    "fsgs_lbs_weights_forward": (c_int, [c_int, c_int, _vp, _vp, _vp, _vp, _vp, _vp]),
    "fsgs_lbs_weights_backward_workspace_bytes": (c_size_t, [c_int, c_int]),
    "fsgs_lbs_weights_backward": (c_int, [c_int, c_int, c_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, c_int,
                                          _vp, c_size_t, _vp]),
    "fsgs_view_pair_counts": (c_int, [POINTER(ViewArgs), _vp, _vp]),
    "fsgs_stage_timing": (c_int, [c_int]),
    "fsgs_stage_times": (c_int, [POINTER(c_float), POINTER(c_int32)]),
    "fsgs_render_pair_counts": (c_int, [POINTER(RenderArgs), _vp, _vp]),
    "fsgs_view_forward": (c_int, [POINTER(ViewArgs), _vp]),
    "fsgs_view_backward": (c_int, [POINTER(ViewArgs), _vp]),
    "fsgs_transmat_forward": (c_int, [c_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "fsgs_transmat_backward": (c_int, [c_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "fsgs_transmat_forward_f64": (c_int, [c_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "fsgs_transmat_backward_f64": (c_int, [c_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "fsgs_lbs_warp_forward": (c_int, [c_int, POINTER(LBS), _vp, _vp, _vp, _vp]),
    "fsgs_lbs_warp_backward": (c_int, [c_int, POINTER(LBS), _vp, _vp, _vp, POINTER(LBSGrads), _vp]),
    "fsgs_preprocess_forward": (c_int, [POINTER(PreprocessArgs), _vp]),
    "fsgs_pack_records": (c_int, [c_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "fsgs_bin_workspace_bytes": (c_size_t, [c_int, c_int, c_int64]),
    "fsgs_bin_tiles": (c_int, [POINTER(BinArgs), _vp]),
    "fsgs_bin_tiles_noalloc": (c_int, [POINTER(BinArgs), _vp]),
    "fsgs_render_forward": (c_int, [POINTER(RenderArgs), _vp]),
    "fsgs_render_backward": (c_int, [POINTER(RenderBwdArgs), _vp]),
    "fsgs_preprocess_backward": (c_int, [POINTER(PreprocessBwdArgs), _vp]),
    "fsgs_sh_factors": (c_int, [c_int, _vp, _vp, _vp, _vp, _vp, _vp, c_int, _vp, _vp, _vp]),
    "fsgs_sh_grad_from_views": (c_int, [c_int, c_int, c_int, c_int, POINTER(c_int32), _vp, c_int64, _vp, _vp, _vp, _vp]),
    "fsgs_compact_workspace_bytes": (c_size_t, [c_int64]),
    "fsgs_compact_plan": (c_int, [c_int64, _vp, _vp, c_size_t, _vp, _vp]),
    "fsgs_compact_rows": (c_int, [c_int, POINTER(RowTensor), c_int64, _vp, _vp, _vp]),
    "fsgs_densify_stats": (c_int, [c_int, _vp, _vp, _vp, _vp, _vp, _vp]),
    "fsgs_densify_select": (c_int, [c_int, _vp, _vp, _vp, c_float, c_float, _vp, _vp]),
    "fsgs_split_children": (c_int, [c_int, c_int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "fsgs_gather_rows": (c_int, [c_int, POINTER(RowTensor), c_int64, _vp, _vp]),
    "fsgs_ssim_forward": (c_int, [c_int, c_int, c_int, c_int, c_float, c_float, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "fsgs_ssim_backward": (c_int, [c_int, c_int, c_int, c_int, c_float, c_float, _vp, _vp, _vp, c_float, c_float,
                                   _vp, _vp, _vp, _vp, _vp]),
    "fsgs_epilogue_forward": (c_int, [c_int, c_int, c_float, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "fsgs_epilogue_backward": (c_int, [c_int, c_int, c_float, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
}

_lib = None


def lib():
    """The loaded library; raises when it has not been built (``python -m fsgs.build``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            raise RuntimeError(f"{LIB} is missing: build it with `python -m fsgs.build` (needs nvcc). "
                               "There is no CPU fallback.")
        handle = ctypes.CDLL(LIB)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)  # AttributeError here = header and library out of sync
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(status, what):
    if status != 0:
        raise RuntimeError(f"{what}: {lib().fsgs_status_string(status).decode()} (status {status})")
