// extern "C" entry points of libbsa_b200.so (declared in include/bsa.h):
// argument validation, kernel-family selection, launch.
#include "common.cuh"

using namespace bsa;

namespace {

int validate_fwd(const bsa_fwd_params* p, const char* who) {
  BSA_CHECK_ARG(p, "%s: null params", who);
  BSA_CHECK_ARG(p->q && p->k && p->v && p->o, "%s: null tensor pointer", who);
  BSA_CHECK_ARG(p->crow && p->col, "%s: null layout pointer", who);
  BSA_CHECK_ARG(p->batch >= 0 && p->hq >= 1 && p->hkv >= 1 && p->d >= 1 && p->sq >= 0 && p->sk >= 0,
                "%s: bad shape batch=%d hq=%d hkv=%d d=%d sq=%d sk=%d", who, p->batch, p->hq, p->hkv,
                p->d, p->sq, p->sk);
  BSA_CHECK_ARG(p->hq % p->hkv == 0, "%s: hq=%d is not a multiple of hkv=%d", who, p->hq, p->hkv);
  BSA_CHECK_ARG(p->h_pat == 1 || p->h_pat == p->hkv || p->h_pat == p->hq,
                "%s: pattern has %d heads, expected 1, %d or %d", who, p->h_pat, p->hkv, p->hq);
  const int bs = p->block_size;
  BSA_CHECK_ARG(bs >= 16 && bs <= 128 && (bs & (bs - 1)) == 0,
                "%s: block_size must be a power of two in [16,128], got %d", who, bs);
  BSA_CHECK_ARG(p->dtype == BSA_F16 || p->dtype == BSA_BF16 || p->dtype == BSA_F32,
                "%s: unknown dtype %d", who, p->dtype);
  BSA_CHECK_ARG(p->row_mode == BSA_ROWS_BY_TILE || p->row_mode == BSA_ROWS_BY_POSITION,
                "%s: unknown row_mode %d", who, p->row_mode);
  BSA_CHECK_ARG((p->q_start == nullptr) == (p->q_end == nullptr) &&
                    (p->k_start == nullptr) == (p->k_end == nullptr),
                "%s: start/end arrays must be given in pairs", who);
  BSA_CHECK_ARG(p->batch <= 65535 && p->hq <= 65535, "%s: batch and hq are limited to 65535", who);
  return BSA_OK;
}

}  // namespace

extern "C" {

int bsa_abi_version(void) { return BSA_ABI_VERSION; }
const char* bsa_last_error(void) { return last_error(); }

int bsa_local_stride_mask(const bsa_local_stride_params* p, uint8_t* mask, void* stream) {
  return layout_local_stride_mask(p, mask, static_cast<cudaStream_t>(stream));
}

int bsa_csr_row_ptr(const uint8_t* mask, int32_t H, int32_t M, int32_t N, int64_t sh, int64_t sm,
                    int64_t sn, int32_t* crow, int32_t* nnz, void* stream) {
  return layout_csr_row_ptr(mask, H, M, N, sh, sm, sn, crow, nnz, static_cast<cudaStream_t>(stream));
}

int bsa_csr_fill_cols(const uint8_t* mask, int32_t H, int32_t M, int32_t N, int64_t sh, int64_t sm,
                      int64_t sn, const int32_t* crow, int32_t* col, int32_t width,
                      int32_t interleave_values, void* stream) {
  return layout_csr_fill_cols(mask, H, M, N, sh, sm, sn, crow, col, width, interleave_values,
                              static_cast<cudaStream_t>(stream));
}

int bsa_fwd_uses_sm100(const bsa_fwd_params* p) {
  int rc = validate_fwd(p, "bsa_fwd_uses_sm100");
  if (rc) return rc;
  if (p->impl == BSA_IMPL_GENERIC) return 0;
  const char* why = nullptr;
  return sm100_fwd_supported(p, &why) ? 1 : 0;
}

int bsa_fwd(const bsa_fwd_params* p, void* stream) {
  int rc = validate_fwd(p, "bsa_fwd");
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (p->impl != BSA_IMPL_GENERIC) {
    const char* why = nullptr;
    if (sm100_fwd_supported(p, &why)) return sm100_fwd(p, s);
    if (p->impl == BSA_IMPL_SM100) {
      set_error("bsa_fwd: the tcgen05 kernel does not serve this call: %s", why ? why : "?");
      return BSA_E_UNSUPPORTED;
    }
  }
  if (p->fine_block != 0) {
    set_error("bsa_fwd: a coarsened fine-block layout (fine_block = %d) is only read by the tcgen05 kernel; "
              "pass the pattern's own layout to the generic kernel", p->fine_block);
    return BSA_E_UNSUPPORTED;
  }
  return generic_fwd(p, s);
}

int bsa_bwd(const bsa_bwd_params* p, void* stream) {
  BSA_CHECK_ARG(p, "bsa_bwd: null params");
  int rc = validate_fwd(&p->f, "bsa_bwd");
  if (rc) return rc;
  BSA_CHECK_ARG(p->f.lse && p->d_o && p->dq && p->dk && p->dv && p->delta && p->ccol && p->row,
                "bsa_bwd: null pointer (lse, dO, dQ, dK, dV, delta and the CSC layout are required)");
  // A pattern with 16- or 32-token blocks coarsened to 64-token blocks (col_bits) is served by the
  // tensor-core kernels only, and only with the dS hand-over: the dK/dV kernel applies the bit masks and the
  // dQ kernel reads the masked dS tiles.
  BSA_CHECK_ARG(p->f.fine_block == 0 || ((p->f.fine_block == 16 || p->f.fine_block == 32) && p->f.col_bits &&
                                         p->ds_ws && p->f.impl != BSA_IMPL_GENERIC),
                "bsa_bwd: a coarsened fine-block layout needs col_bits, a dS workspace and the tensor-core kernels; "
                "pass the pattern's own layout otherwise");
  BSA_CHECK_ARG(!p->f.q_start && !p->f.k_start && p->f.row_mode == BSA_ROWS_BY_TILE,
                "bsa_bwd: padded / packed batches have no backward "
                "(as in dkernel/ops/__init__.py:57-58,79-80)");
  if (p->ds_ws)
    BSA_CHECK_ARG(p->csc_csr && p->ds_tiles_per_head > 0 && reinterpret_cast<uintptr_t>(p->ds_ws) % 128 == 0 &&
                      p->ds_tiles_per_head * 64 < (1ll << 31),
                  "bsa_bwd: a dS workspace needs csc_csr, ds_tiles_per_head in (0, 2^25) and 128-byte alignment");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (p->f.impl != BSA_IMPL_GENERIC) {
    const char* why = nullptr;
    if (sm100_bwd_supported(p, &why)) return sm100_bwd(p, s);
    if (p->f.impl == BSA_IMPL_SM100 || p->f.fine_block != 0) {
      set_error("bsa_bwd: the tcgen05 kernel does not serve this call: %s", why ? why : "?");
      return BSA_E_UNSUPPORTED;
    }
  }
  return generic_bwd(p, s);
}

size_t bsa_decode_workspace_bytes(const bsa_decode_params* p) {
  if (!p) return 0;
  return decode_workspace_bytes(p);
}

int bsa_decode(const bsa_decode_params* p, void* stream) {
  return decode_run(p, static_cast<cudaStream_t>(stream));
}

int bsa_decode_static(const bsa_decode_params* p, void* stream) {
  return decode_run_static(p, static_cast<cudaStream_t>(stream));
}

size_t bsa_decode_static_capacity(void) { return decode_static_capacity(); }

int bsa_merge_partials(const void* o_parts, const float* lse_parts, int32_t P, int64_t rows,
                       int32_t d, int64_t part_stride_o, int64_t row_stride_o,
                       int64_t part_stride_lse, int64_t row_stride_lse, void* o,
                       int64_t o_row_stride, float* lse, int32_t dtype, void* stream) {
  return merge_partials(o_parts, lse_parts, P, rows, d, part_stride_o, row_stride_o,
                        part_stride_lse, row_stride_lse, o, o_row_stride, lse, dtype,
                        static_cast<cudaStream_t>(stream));
}

size_t bsa_xchg_buffer_bytes(int32_t world, int64_t rows, int32_t d) {
  return xchg_buffer_bytes(world, rows, d);
}

int bsa_xchg_merge(const bsa_xchg_params* p, void* stream) {
  return xchg_merge(p, static_cast<cudaStream_t>(stream));
}

int bsa_wait_status(int32_t* status, int32_t reset) { return read_wait_status(status, reset); }

int bsa_set_wait_status_mirror(int32_t* host_word) { return set_wait_status_mirror(host_word); }

int bsa_selftest_wait_timeout(uint32_t limit_us, void* stream) {
  return selftest_wait_timeout(limit_us, static_cast<cudaStream_t>(stream));
}

const char* bsa_fwd_why_not_sm100(const bsa_fwd_params* p) {
  if (validate_fwd(p, "bsa_fwd_why_not_sm100")) return last_error();
  const char* why = nullptr;
  if (sm100_fwd_supported(p, &why)) return nullptr;
  return why ? why : "unsupported";
}

}  // extern "C"
