// Shared host/device helpers for the block-sparse attention library.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/bsa.h"

namespace bsa {

// ---- error reporting (thread-local text, fetched through bsa_last_error) ----
void set_error(const char* fmt, ...);
const char* last_error();

#define BSA_CHECK_ARG(cond, ...)                    \
  do {                                              \
    if (!(cond)) {                                  \
      ::bsa::set_error(__VA_ARGS__);                \
      return BSA_E_BADARG;                          \
    }                                               \
  } while (0)

#define BSA_CHECK_CUDA(expr)                                                      \
  do {                                                                            \
    cudaError_t _e = (expr);                                                      \
    if (_e != cudaSuccess) {                                                      \
      ::bsa::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),    \
                       __FILE__, __LINE__);                                       \
      return BSA_E_CUDA;                                                          \
    }                                                                             \
  } while (0)

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("launch of %s failed: %s", what, cudaGetErrorString(e));
    return BSA_E_CUDA;
  }
  return BSA_OK;
}

// ---- element types ----
template <typename T> struct Elem;
template <> struct Elem<__half> {
  static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
};
template <> struct Elem<float> {
  static __device__ __forceinline__ float to_f(float x) { return x; }
  static __device__ __forceinline__ float from_f(float x) { return x; }
};

inline size_t dtype_size(int dtype) { return dtype == BSA_F32 ? 4 : 2; }

__host__ __device__ inline int cdiv_i(int a, int b) { return (a + b - 1) / b; }

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// pattern head serving q head h: one shared pattern, one per kv head, or one per q head
__host__ __device__ inline int pattern_head(int h, int h_pat, int hq, int hkv) {
  return h_pat == 1 ? 0 : (h_pat == hq ? h : h / (hq / hkv));
}

// entry points implemented in the per-kernel translation units
int layout_local_stride_mask(const bsa_local_stride_params* p, uint8_t* mask, cudaStream_t s);
int layout_csr_row_ptr(const uint8_t* mask, int H, int M, int N, int64_t sh, int64_t sm, int64_t sn,
                       int32_t* crow, int32_t* nnz, cudaStream_t s);
int layout_csr_fill_cols(const uint8_t* mask, int H, int M, int N, int64_t sh, int64_t sm, int64_t sn,
                         const int32_t* crow, int32_t* col, int width, int interleave, cudaStream_t s);
int generic_fwd(const bsa_fwd_params* p, cudaStream_t s);
int generic_bwd(const bsa_bwd_params* p, cudaStream_t s);
bool sm100_fwd_supported(const bsa_fwd_params* p, const char** why);
int sm100_fwd(const bsa_fwd_params* p, cudaStream_t s);
bool sm100_bwd_supported(const bsa_bwd_params* p, const char** why);
int sm100_bwd(const bsa_bwd_params* p, cudaStream_t s);
size_t decode_workspace_bytes(const bsa_decode_params* p);
int decode_run(const bsa_decode_params* p, cudaStream_t s);
int decode_run_static(const bsa_decode_params* p, cudaStream_t s);
size_t decode_static_capacity();
int merge_partials(const void* o_parts, const float* lse_parts, int P, int64_t rows, int d,
                   int64_t pso, int64_t rso, int64_t psl, int64_t rsl, void* o, int64_t ors,
                   float* lse, int dtype, cudaStream_t s);
size_t xchg_buffer_bytes(int world, int64_t rows, int d);
int xchg_merge(const bsa_xchg_params* p, cudaStream_t s);
int read_wait_status(int* out, int reset);
int set_wait_status_mirror(int* host_word);
int selftest_wait_timeout(uint32_t limit_us, cudaStream_t s);
int* wait_status_ptr();

}  // namespace bsa
