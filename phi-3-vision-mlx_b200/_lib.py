"""ctypes binding of libphi3b200.so (the C ABI declared in include/phi3_b200.h).

There is deliberately NO fallback: if the shared library is missing or a call fails, this
module raises. Build with `python -c "import __graft_entry__ as g; g.build()"` or
`make -C phi-3-vision-mlx_b200/csrc`.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# Two builds of the same sources: the full library, and the language-model subset (no Phi-3 attention / vision / quantisation
# kernels) that a fresh checkout compiles when only an engine model is served. The full one wins when both exist.
FULL_PATH = os.path.join(_HERE, 'libphi3b200.so')
LM_PATH = os.path.join(_HERE, 'libphi3b200_lm.so')
LIB_PATH = os.environ.get('P3_LIB') or FULL_PATH                               # P3_LIB: tuning builds (tools/), same ABI


def ensure_built(full=True):
    """compile the CUDA library if no usable build is there (make -C csrc; sm_100a, needs nvcc): the full library, or with
    full=False just the subset the engine models use. Existing builds are never rebuilt here."""
    import subprocess
    if os.environ.get('P3_LIB') or os.path.exists(FULL_PATH) or (not full and os.path.exists(LM_PATH)):
        return
    env = dict(os.environ)
    if not any(os.path.exists(os.path.join(d, 'nvcc')) for d in env.get('PATH', '').split(os.pathsep) if d):
        env['PATH'] = env.get('PATH', '') + os.pathsep + '/usr/local/cuda/bin'
    subprocess.check_call(['make', '-C', os.path.join(_HERE, 'csrc'), '-j8', 'all' if full else 'lm'], env=env,
                          stdout=subprocess.DEVNULL)


EPI_NONE, EPI_QGELU, EPI_GELU, EPI_RESIDUAL, EPI_SWIGLU, EPI_F32, EPI_RESIDUAL_F32 = range(7)
EPI_ROPE_KV = 8
GEMM_WPLAN_BYTES = 320
PAGE = 64

_p, _i, _l, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float
_SIGS = {
    'p3_embed_gather': [_p, _p, _p, _l, _i, _i, _p, _p],
    'p3_rmsnorm': [_p, _p, _p, _l, _i, _f, _p],
    'p3_layernorm': [_p, _p, _p, _p, _l, _i, _f, _i, _p],
    'p3_rope_kvwrite': [_p, _p, _p, _l, _i, _i, _i, _i, _i, _i, _i, _p, _p, _i, _i, _p, _p],
    'p3_row_stats': [_p, _l, _l, _i, _p, _p, _p, _i, _p, _p, _i, _p, _p, _p],
    'p3_gemm_skinny': [_p, _l, _p, _f, _p, _p, _l, _p, _i, _i, _i, _i, _p, _i, _p, _p, _l, _p],
    'p3_gemm_skinny_qkv_rope': [_p, _l, _p, _f, _p, _p, _p, _i, _p, _p, _l, _i, _i, _i, _i, _i, _i, _i, _p, _i, _p, _p, _i, _i, _p, _l, _p],
    'p3_gemm_skinny_w4': [_p, _l, _p, _f, _p, _p, _p, _l, _p, _i, _i, _i, _i, _p, _i, _p, _p, _l, _p],
    'p3_gemm_skinny_qkv_rope_w4': [_p, _l, _p, _f, _p, _p, _p, _p, _i, _p, _p, _l, _i, _i, _i, _i, _i, _i, _i, _p, _i, _p, _p, _i, _i, _p, _l, _p],
    'p3_gemm': [_p, _l, _p, _l, _p, _p, _l, _p, _p, _l, _i, _i, _i, _i, _p],
    'p3_attention_prefill': [_p, _p, _p, _l, _l, _l, _p, _l, _i, _i, _i, _i, _i, _f, _i, _i, _p, _p, _p, _i, _i, _p],
    'p3_attention_decode': [_p, _p, _p, _l, _l, _l, _p, _l, _i, _i, _i, _i, _i, _f, _i, _p, _p, _p, _i, _i, _i, _p, _p, _p, _l, _p],
    'p3_attention_decode_q4': [_p, _p, _p, _l, _l, _l, _p, _l, _i, _i, _i, _i, _i, _f, _i, _i, _p, _p, _p, _p, _p, _i,
                               _i, _i, _p, _p, _p, _l, _p],
    'p3_kv_quantize_q4g32': [_p, _p, _p, _p, _i, _i, _i, _i, _i, _p],
    'p3_top_p_sample': [_p, _l, _l, _i, _f, _f, _p, _p, _p, _p, _l, _p],
    'p3_decode_advance': [_p, _p, _l, _i, _p, _p, _p, _p],
    'p3_hd_resize_h': [_p, _l, _l, _i, _i, _p, _i, _p, _p, _i, _p],
    'p3_hd_resize_v_pad': [_p, _i, _i, _i, _p, _p, _i, _i, _i, _i, _p, _p],
    'p3_hd_tile_crops': [_p, _i, _i, _p, _p, _p, _p, _p, _p, _p],
    'p3_patch_im2col': [_p, _p, _i, _i, _p],
    'p3_clip_embed': [_p, _p, _p, _p, _i, _i, _p],
    'p3_gn_assemble': [_p, _p, _p, _p, _i, _i, _i, _p],
    'p3_mega_pack': [_p, _p, _i, _i, _i, _i, _i, _i, _p],
    'p3_row_sumsq': [_p, _l, _p, _l, _i, _p],
    'p3_rope_table': [_p, _l, _i, _p, _p, _p, _i, _i, _i, _f, _p],
    'p3_embed_gather_xg': [_p, _p, _p, _l, _i, _i, _p, _p, _p, _p],
    # decoders with an fp32 residual stream over a shared page pool (csrc/seq_ops.cu)
    'p3_embed_rows_f32': [_p, _p, _p, _p, _i, _l, _i, _i, _f, _l, _p],
    'p3_postnorm_residual': [_p, _l, _p, _p, _p, _p, _i, _l, _i, _f, _p],
    'p3_rmsnorm_rows_f32': [_p, _p, _p, _p, _i, _l, _i, _f, _p],
    'p3_glu_clamped': [_p, _l, _p, _l, _i, _l, _i, _f, _f, _p, _p],
    'p3_router_topk': [_p, _l, _i, _p, _p, _i, _i, _i, _i, _p, _p, _p],
    'p3_moe_sort': [_p, _i, _i, _p, _p, _p, _p],
    'p3_moe_combine': [_p, _l, _p, _p, _i, _p, _l, _i, _p],
    'p3_gather_rows': [_p, _l, _i, _p, _i, _p, _l, _i, _p],
    'p3_distance_penalty_table': [_p, _p, _p, _i, _i, _p],
    # single-norm parallel layers, latent-vector attention, sigmoid group routing (csrc/seq_ops.cu)
    'p3_residual_layernorm': [_p, _p, _l, _p, _l, _p, _p, _p, _p, _l, _p, _l, _i, _l, _i, _f, _p],
    'p3_glu_silu': [_p, _p, _l, _p, _l, _i, _l, _i, _p],
    'p3_router_sigmoid_groups': [_p, _l, _i, _p, _p, _p, _l, _i, _i, _i, _i, _i, _i, _f, _p, _p, _p],
    'p3_logit_softcap': [_p, _l, _f, _f, _p],
    # sandwich norms, token shift, relu^2 unit, softmax group router with identity experts, head norm of a recurrent mixer
    # (csrc/seq_ops.cu, csrc/recurrent.cu)
    'p3_postnorm_prenorm': [_p, _l, _p, _p, _p, _p, _p, _p, _i, _l, _i, _f, _p],
    'p3_token_shift': [_p, _p, _p, _p, _p, _p, _p, _i, _l, _i, _p],
    'p3_relu2': [_p, _l, _p, _l, _p, _l, _i, _l, _i, _p],
    'p3_router_groups': [_p, _l, _p, _i, _i, _i, _i, _i, _f, _i, _p, _p, _p],
    'p3_moe_combine_identity': [_p, _l, _p, _p, _p, _i, _i, _p, _p, _l, _p, _l, _i, _p],
    'p3_headnorm_gate': [_p, _l, _p, _i, _i, _p, _p, _l, _f, _f, _p, _l, _i, _l, _p],
    # hashed token-pair embedding, linear distance bias, head norm with a shared gain / silu gate (csrc/seq_ops.cu, csrc/recurrent.cu)
    'p3_embed_pair_rows_f32': [_p, _p, _p, _p, _p, _p, _p, _l, _p, _l, _i, _i, _f, _l, _l, _l, _p],
    'p3_distance_linear_table': [_p, _p, _i, _i, _p],
    'p3_headnorm_gate_x': [_p, _l, _p, _i, _i, _p, _i, _p, _l, _i, _f, _f, _p, _l, _i, _l, _p],
}
ROUTER_SOFTMAX, ROUTER_GROUP_MAX, ROUTER_PLAIN_WEIGHTS = 1, 2, 4          # mode bits of p3_router_groups
_STRUCT_ENTRIES = ['p3_gemm_any', 'p3_qkv_post', 'p3_attn_window_prefill', 'p3_attn_window_decode', 'p3_latent_post',
                   'p3_qkv_rope_post', 'p3_matrix_memory_scan', 'p3_gla_scan']
ATTN_WINDOW_MMA = os.environ.get('P3_ATTN_WINDOW_MMA', '1') != '0'

_lib = None
launches = 0          # number of p3_* kernel-launching calls issued (bench.py reports it)


def exported_symbols():
    return sorted(list(_SIGS) + ['p3_last_error', 'p3_version', 'p3_attention_decode_workspace', 'p3_decode_mega',
                                 'p3_decode_mega_ctas', 'p3_gemm_fused', 'p3_gemm_plan_weights', 'p3_gemm_skinny_x', 'p3_trace_set', 'p3_trace_count',
                                 'p3_attn_window_tile_rows', 'p3_matrix_memory_state_floats', 'p3_gla_state_floats']
                  + _STRUCT_ENTRIES)


def lib():
    global _lib
    if _lib is None:
        path = LIB_PATH if os.path.exists(LIB_PATH) else LM_PATH
        if not os.path.exists(path):
            raise RuntimeError(f'{LIB_PATH} is missing: the CUDA extension must be built (no CPU fallback exists). '
                               'Run __graft_entry__.build().')
        L = C.CDLL(path)
        lm_only = not hasattr(L, 'p3_attention_decode')
        for name, sig in _SIGS.items():
            if lm_only and not hasattr(L, name):
                continue                                     # subset build: calling a missing entry raises AttributeError
            fn = getattr(L, name)
            fn.argtypes, fn.restype = sig, C.c_int
        if lm_only:
            for name in _STRUCT_ENTRIES:
                getattr(L, name).argtypes, getattr(L, name).restype = [_p, _p], C.c_int
            L.p3_attn_window_tile_rows.argtypes, L.p3_attn_window_tile_rows.restype = [_p], C.c_int
            L.p3_matrix_memory_state_floats.argtypes, L.p3_matrix_memory_state_floats.restype = [_i, _i, _i], C.c_int64
            L.p3_gla_state_floats.argtypes, L.p3_gla_state_floats.restype = [_i, _i, _i], C.c_int64
            L.p3_last_error.restype = C.c_char_p
            L.p3_version.restype = C.c_int
            _lib = L
            return _lib
        L.p3_last_error.restype = C.c_char_p
        L.p3_version.restype = C.c_int
        L.p3_attention_decode_workspace.argtypes = [_i, _i, _i, _i, _i]
        L.p3_attention_decode_workspace.restype = C.c_int64
        L.p3_decode_mega.argtypes, L.p3_decode_mega.restype = [_p, _p], C.c_int      # (const p3_mega_args*, stream)
        L.p3_decode_mega_ctas.argtypes, L.p3_decode_mega_ctas.restype = [], C.c_int
        L.p3_gemm_fused.argtypes, L.p3_gemm_fused.restype = [_p, _p], C.c_int        # (const p3_gemm_args*, stream)
        L.p3_gemm_plan_weights.argtypes, L.p3_gemm_plan_weights.restype = [_p, _l, _i, _i, _p], C.c_int
        L.p3_gemm_skinny_x.argtypes, L.p3_gemm_skinny_x.restype = [_p, _p], C.c_int        # (const p3_skinny_args*, stream)
        L.p3_trace_set.argtypes, L.p3_trace_set.restype = [_p, C.c_int], C.c_int           # diagnostics (tools/chain_trace.py)
        L.p3_trace_count.argtypes, L.p3_trace_count.restype = [], C.c_int
        for name in _STRUCT_ENTRIES:                                                        # (const args*, stream)
            getattr(L, name).argtypes, getattr(L, name).restype = [_p, _p], C.c_int
        L.p3_attn_window_tile_rows.argtypes, L.p3_attn_window_tile_rows.restype = [_p], C.c_int
        L.p3_matrix_memory_state_floats.argtypes, L.p3_matrix_memory_state_floats.restype = [_i, _i, _i], C.c_int64
        L.p3_gla_state_floats.argtypes, L.p3_gla_state_floats.restype = [_i, _i, _i], C.c_int64
        _lib = L
    return _lib


def ptr(t):
    """Device (or host) address of a torch tensor, None -> NULL."""
    return None if t is None else t.data_ptr()


def call(name, *args):
    global launches
    L = lib()
    if len(args) != len(_SIGS[name]):
        raise TypeError(f'{name}: expected {len(_SIGS[name])} arguments, got {len(args)}')
    rc = getattr(L, name)(*args)
    launches += 1
    if rc != 0:
        raise RuntimeError(f'{name} failed ({rc}): {L.p3_last_error().decode()}')


def call_struct(name, args_struct, stream):
    """Entries that take one plain-old-data argument struct (include/phi3_b200.h) + the stream."""
    global launches
    L = lib()
    rc = getattr(L, name)(C.byref(args_struct), stream)
    launches += 1
    if rc != 0:
        raise RuntimeError(f'{name} failed ({rc}): {L.p3_last_error().decode()}')


class GemmArgs(C.Structure):
    """p3_gemm_args (include/phi3_b200.h)"""
    _fields_ = [('X', _p), ('ldx', _l), ('W', _p), ('ldw', _l), ('bias', _p), ('out', _p), ('ldo', _l), ('resid', _p),
                ('row_map', _p), ('M', _l), ('N', C.c_int32), ('K', C.c_int32), ('epi', C.c_int32), ('impl', C.c_int32),
                ('ss_in', _p), ('n_ss_in', C.c_int32), ('eps', C.c_float), ('ss_out', _p), ('w_plan', _p),
                ('cosT', _p), ('sinT', _p), ('tab_bstride', _l),
                ('L', C.c_int32), ('n_heads', C.c_int32), ('n_kv', C.c_int32), ('hd', C.c_int32), ('past', C.c_int32),
                ('row_div', C.c_int32), ('write_cache', C.c_int32), ('bt_stride', C.c_int32),
                ('past_dev', _p), ('pool', _p), ('block_table', _p), ('splitk_ws', _p), ('splitk_ws_bytes', _l)]


class SkinnyArgs(C.Structure):
    """p3_skinny_args (include/phi3_b200.h)"""
    _fields_ = [('op', C.c_int32), ('X', _p), ('ldx', _l), ('norm_w', _p), ('eps', C.c_float), ('W', _p), ('Wq', _p), ('Wmeta', _p),
                ('out', _p), ('ldo', _l), ('resid', _p), ('M', C.c_int32), ('N', C.c_int32), ('K', C.c_int32), ('epi', C.c_int32),
                ('ss_in', _p), ('n_ss_in', C.c_int32), ('ss_out', _p), ('l2_prefetch', _p), ('l2_prefetch_bytes', _l),
                ('xg_gain', _p), ('xg_out', _p), ('ldxg', _l), ('rs_epi', C.c_int32),
                ('cosT', _p), ('sinT', _p), ('tab_bstride', _l),
                ('B', C.c_int32), ('L', C.c_int32), ('n_heads', C.c_int32), ('n_kv', C.c_int32), ('hd', C.c_int32), ('past', C.c_int32),
                ('row_div', C.c_int32), ('bt_stride', C.c_int32), ('write_cache', C.c_int32),
                ('past_dev', _p), ('pool', _p), ('block_table', _p), ('packed', C.c_int32)]


class WeightPlan:
    """caller-owned, 64-byte aligned blob holding the TMA descriptors of one weight matrix (p3_gemm_plan_weights)"""

    def __init__(self, w):
        self._raw = C.create_string_buffer(GEMM_WPLAN_BYTES + 64)
        self.addr = (C.addressof(self._raw) + 63) & ~63
        self.w = w                                             # keeps the tensor (and its address) alive
        rc = lib().p3_gemm_plan_weights(w.data_ptr(), w.stride(0), w.shape[0], w.shape[1], self.addr)
        if rc != 0:
            raise RuntimeError(f'p3_gemm_plan_weights failed ({rc}): {lib().p3_last_error().decode()}')


class GemmAnyArgs(C.Structure):
    """p3_gemm_any_args (include/phi3_b200.h)"""
    _fields_ = [('X', _p), ('ldx', _l), ('x_f32', C.c_int32), ('x_rows', _p), ('x_row_div', C.c_int32),
                ('W', _p), ('ldw', _l), ('w_f32', C.c_int32), ('w_group_stride', _l),
                ('bias', _p), ('bias_group_stride', _l), ('out', _p), ('ldo', _l), ('out_f32', C.c_int32),
                ('M', _l), ('N', C.c_int32), ('K', C.c_int32), ('seg_offsets', _p), ('n_groups', C.c_int32),
                ('force_fma', C.c_int32),
                ('n_batch', C.c_int32), ('x_batch_stride', _l), ('w_batch_stride', _l), ('out_batch_stride', _l),
                ('gate', _p), ('ld_gate', _l)]


class QkvPostArgs(C.Structure):
    """p3_qkv_post_args (include/phi3_b200.h)"""
    _fields_ = [('proj', _p), ('ld_proj', _l), ('q_off', C.c_int32), ('k_off', C.c_int32), ('v_off', C.c_int32), ('g_off', C.c_int32),
                ('n_heads', C.c_int32), ('n_kv', C.c_int32), ('dim', C.c_int32), ('vdim', C.c_int32),
                ('q_gain', _p), ('k_gain', _p), ('eps', C.c_float),
                ('v_first', _p), ('v_mode', C.c_int32), ('v_lambda', C.c_float),
                ('q_out', _p), ('ld_q', _l), ('gate_out', _p),
                ('k_pool', _p), ('v_pool', _p), ('block_table', _p), ('bt_stride', C.c_int32),
                ('tok_slot', _p), ('tok_pos', _p), ('T', C.c_int32), ('act_f32', C.c_int32), ('cache_f32', C.c_int32),
                ('bias', _p), ('q_temp_coef', C.c_float), ('q_temp_every', C.c_int32)]


class AttnWindowArgs(C.Structure):
    """p3_attn_window_args (include/phi3_b200.h)"""
    _fields_ = [('q', _p), ('ld_q', _l), ('k_pool', _p), ('v_pool', _p), ('block_table', _p), ('bt_stride', C.c_int32),
                ('sink', _p), ('penalty', _p), ('n_penalty', C.c_int32), ('gate', _p), ('out', _p), ('ld_out', _l),
                ('n_heads', C.c_int32), ('n_kv', C.c_int32), ('dim', C.c_int32), ('vdim', C.c_int32), ('scale', C.c_float),
                ('window', C.c_int32), ('act_f32', C.c_int32), ('cache_f32', C.c_int32), ('tiles', _p), ('n_tiles', C.c_int32),
                ('n_splits', C.c_int32), ('ws', _p), ('v_ld', C.c_int32), ('keep_first', C.c_int32), ('sig_bias', _p),
                ('out_scale', C.c_float), ('elem_gate', _p), ('ld_elem_gate', _l)]


class LatentPostArgs(C.Structure):
    """p3_latent_post_args (include/phi3_b200.h)"""
    _fields_ = [('proj', _p), ('ld_proj', _l), ('q_off', C.c_int32), ('c_off', C.c_int32), ('gate_off', C.c_int32), ('up_off', C.c_int32),
                ('n_heads', C.c_int32), ('dim', C.c_int32), ('rot_dim', C.c_int32), ('kv_rank', C.c_int32), ('rot_n', C.c_int32),
                ('n_ff', C.c_int32),
                ('c_gain', _p), ('eps', C.c_float), ('freq', _p), ('rot_mag', C.c_float),
                ('q_plain', _p), ('ld_qp', _l), ('q_lat', _p), ('ld_ql', _l), ('hid', _p), ('ld_hid', _l), ('hid_off', C.c_int32),
                ('cache', _p), ('block_table', _p), ('bt_stride', C.c_int32),
                ('tok_slot', _p), ('tok_pos', _p), ('T', C.c_int32), ('act_f32', C.c_int32), ('cache_f32', C.c_int32),
                ('pair_mode', C.c_int32), ('q_src', _p), ('ld_qsrc', _l), ('cq_off', C.c_int32), ('q_rank', C.c_int32),
                ('cq_gain', _p), ('cq_out', _p), ('ld_cq', _l)]


class QkvRopePostArgs(C.Structure):
    """p3_qkv_rope_post_args (include/phi3_b200.h)"""
    _fields_ = [('proj', _p), ('ld_proj', _l), ('q_off', C.c_int32), ('k_off', C.c_int32), ('v_off', C.c_int32), ('bias', _p),
                ('n_heads', C.c_int32), ('n_kv', C.c_int32), ('dim', C.c_int32), ('vdim', C.c_int32), ('rot_n', C.c_int32),
                ('freq', _p), ('q_out', _p), ('ld_q', _l),
                ('k_pool', _p), ('v_pool', _p), ('block_table', _p), ('bt_stride', C.c_int32),
                ('tok_slot', _p), ('tok_pos', _p), ('T', C.c_int32), ('act_f32', C.c_int32), ('cache_f32', C.c_int32)]


class MatrixMemoryArgs(C.Structure):
    """p3_matrix_memory_args (include/phi3_b200.h)"""
    _fields_ = [('proj', _p), ('ld_proj', _l), ('q_off', C.c_int32), ('k_off', C.c_int32), ('v_off', C.c_int32),
                ('i_off', C.c_int32), ('f_off', C.c_int32), ('i_bias', _p), ('f_bias', _p),
                ('n_heads', C.c_int32), ('dim', C.c_int32), ('vdim', C.c_int32), ('q_scale', C.c_float), ('gate_cap', C.c_float),
                ('state', _p), ('seqs', _p), ('n_seqs', C.c_int32), ('out', _p), ('ld_out', _l), ('den', _p), ('rs_force', C.c_int32)]


class GlaArgs(C.Structure):
    """p3_gla_args (include/phi3_b200.h)"""
    _fields_ = [('proj', _p), ('ld_proj', _l), ('q_off', C.c_int32), ('k_off', C.c_int32), ('v_off', C.c_int32),
                ('z', _p), ('ld_z', _l), ('z_bias', _p), ('inv_tau', C.c_float),
                ('n_heads', C.c_int32), ('dim', C.c_int32), ('vdim', C.c_int32), ('q_scale', C.c_float),
                ('state', _p), ('seqs', _p), ('n_seqs', C.c_int32), ('out', _p), ('ld_out', _l), ('rs_force', C.c_int32),
                ('n_rows', C.c_int32), ('lr', _p), ('ld_lr', _l), ('a2', _p), ('rank', C.c_int32)]
