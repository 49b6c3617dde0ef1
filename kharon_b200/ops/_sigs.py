"""ctypes prototypes of the CUDA kernel library (``libkharon_cuda.so``)."""
import ctypes as C

i32, i64, f32, u32 = C.c_int32, C.c_int64, C.c_float, C.c_uint32
vp, cp, long_ = C.c_void_p, C.c_char_p, C.c_long


def _sig(lib, name, res, *args):
    fn = getattr(lib, name)
    fn.restype = res
    fn.argtypes = list(args)


def declare(lib):
    _sig(lib, "kh_cuda_last_error", cp)
    _sig(lib, "kh_cuda_error_word", i32, i32)
    _sig(lib, "kh_gemm_bf16", i32, vp, i32, i32, vp, i32, i32, vp, i32, i32, i32, i32, i32, i32, i32, vp, vp,
         i32, f32, i32, i32, vp)
    _sig(lib, "kh_gemm_bf16_colsum", i32, vp, i32, i32, vp, i32, i32, vp, i32, i32, i32, i32, i32, i32, i32, vp, vp,
         i32, f32, i32, i32, vp, vp)
    _sig(lib, "kh_embed_fwd", i32, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp)
    _sig(lib, "kh_embed_bwd", i32, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp)
    _sig(lib, "kh_colsum", i32, vp, i32, vp, vp, i32, i32, i32, vp)
    _sig(lib, "kh_colsum_scratch_elems", long_, i32, i32)
    _sig(lib, "kh_layernorm_fwd", i32, vp, vp, vp, vp, vp, vp, i32, i32, vp)
    _sig(lib, "kh_layernorm_bwd_scratch_elems", long_, i32, i32)
    _sig(lib, "kh_layernorm_bwd", i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, vp)
    _sig(lib, "kh_xent", i32, vp, i32, i32, vp, vp, f32, vp, vp, i32, i32, vp)
    _sig(lib, "kh_sum_f32", i32, vp, long_, f32, vp, i32, vp)
    _sig(lib, "kh_adamw", i32, vp, vp, vp, vp, vp, long_, f32, f32, f32, f32, f32, f32, f32, f32, i32, vp)
    _sig(lib, "kh_cast_f32_bf16", i32, vp, vp, long_, vp)
    _sig(lib, "kh_add_bf16", i32, vp, vp, vp, long_, vp)
    _sig(lib, "kh_fill_u32", i32, vp, long_, u32, vp)
    for name, proto in _OPTIONAL.items():
        if hasattr(lib, name):
            _sig(lib, name, *proto)


# entry points that live in translation units added after the first ones; declared when present
_OPTIONAL = {
    "kh_gemm_f32": (i32, vp, long_, long_, vp, long_, long_, vp, long_, i32, i32, i32, vp),
    "kh_grpo_advantages_dev": (i32, vp, vp, i32, i32, f32, vp),
    "kh_grpo_coef_dev": (i32, vp, vp, vp, vp, i32, i32, i32, i32, f32, vp),
    "kh_xent_stats": (i32, vp, i32, i32, vp, i32, vp, i32, vp),
    "kh_xent_grad": (i32, vp, i32, i32, vp, i32, vp, vp, vp, f32, i32, vp),
    "kh_wait_probe": (i32, vp, u32, u32, vp, vp),
    "kh_gemm_skinny": (i32, vp, i32, vp, i32, vp, i32, i32, i32, i32, i32, vp, vp, i32, vp, vp, vp, vp),
    "kh_gemm_skinny2": (i32, vp, i32, vp, i32, vp, i32, i32, i32, i32, i32, vp, vp, i32, vp, vp, vp, i32, vp),
    "kh_gemm_skinny_scratch_elems": (long_, i32, i32, i32),
    "kh_zero1_step": (i32, vp, vp, vp, vp, vp, vp, long_, i32, i32, f32, f32, f32, f32, f32, f32, f32, u32, i32, vp),
    "kh_gemm_comm": (i32, vp, i32, i32, vp, i32, i32, vp, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp, vp, u32, u32,
                     C.c_uint64, vp, vp, vp, vp, i32, i32, vp, i32, i32, vp),
    "kh_vp_combine": (i32, vp, vp, vp, C.c_uint64, vp, vp, vp, vp, i32, i32, i32, vp),
    "kh_tmap_cache_limit": (long_, long_),
    "kh_zero1_max_grid": (i32,),
    "kh_set_pdl": (i32, i32),
    "kh_set_peer_wait_limit_ms": (long_, long_),
    "kh_p2p_put": (i32, vp, vp, C.c_longlong, vp, vp, vp),
    "kh_p2p_wait": (i32, vp, vp, u32, vp),
    "kh_append_kv": (i32, vp, i32, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp),
    "kh_decode_layers_ok": (i32, i32, i32, i32, i32, i32),
    "kh_decode_layers": (i32, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, long_, vp, vp, vp, i32, i32, i32, f32,
                         vp, vp, vp, vp, i32, i32, vp, i32, vp, vp),
    "kh_paged_attn_split": (i32, vp, i32, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, f32, i32, i32, i32, i32, vp),
    "kh_paged_attn": (i32, vp, i32, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, f32, i32, i32, i32, vp),
    "kh_gather_rows": (i32, vp, vp, vp, i32, i32, vp),
    "kh_copy_blocks": (i32, vp, vp, vp, i32, i32, long_, long_, vp),
    "kh_sample2": (i32, vp, i32, i32, f32, C.c_uint64, i32, vp, i32, vp, i32, vp),
    "kh_sample": (i32, vp, i32, i32, f32, C.c_uint64, i32, i32, vp, i32, vp),
    "kh_flash_fwd": (i32, vp, vp, vp, i32, i32, i32, i32, i32, f32, vp),
    "kh_flash_bwd": (i32, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, f32, vp),
}
