// extern "C" entry points that are pure dispatch (declared in include/sphconv_b200.h).
#include <stdarg.h>
#include <string.h>

#include <atomic>

#include "common.cuh"

namespace sph {

static thread_local char g_err[512] = "";
static std::atomic<long long> g_launches{0};

void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int current_sm_count() {
  constexpr int kMaxDev = 64;
  static std::atomic<int> s_sms[kMaxDev];     // zero-initialised; a racing first call writes the same value twice
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    set_error("current_sm_count: cudaGetDevice failed");
    return 0;
  }
  int n = (dev >= 0 && dev < kMaxDev) ? s_sms[dev].load(std::memory_order_relaxed) : 0;
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      set_error("current_sm_count: cudaDeviceGetAttribute failed");
      return 0;
    }
    if (dev >= 0 && dev < kMaxDev) s_sms[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

// conv_generic.cu
int conv_gather_generic(const void* rows, int dtype, int64_t n_rows, const void* weight, const int* nbr,
                        int64_t n_out, int kv, int K, int N, int flip_k, const float* scale, const float* bias,
                        int relu, void* out, int out_dtype, int* status, cudaStream_t st);
int conv_wgrad_generic(const void* rows, const void* dout, int dtype, int64_t n_rows, const int* nbr,
                       int64_t n_out, int kv, int K, int N, float* dw, int* status, cudaStream_t st);
// conv_tc.cu
int conv_gather_tc(const void* rows, int dtype, int64_t n_rows, const void* packed, const int* nbr, int64_t n_out,
                   int kv, int K, int N, int flip_k, const float* scale, const float* bias, int relu, void* out,
                   int out_dtype, int* status, cudaStream_t st);
bool conv_tc_supported(int dtype, int kv, int K, int N);
int64_t packed_weight_bytes(int dtype, int kv, int K, int N);
int pack_weight(const void* w, int dtype, int kv, int K, int N, void* packed, cudaStream_t st);
// conv_tc_rows.cu
bool conv_tc_rows_supported(int dtype, int kv, int K, int N);
int conv_gather_tc_rows(const void* rows, int dtype, int64_t n_rows, const void* packed, const int* nbr, int64_t n_out,
                        int kv, int K, int N, int flip_k, const float* scale, const float* bias, int relu, void* out,
                        int out_dtype, int* status, cudaStream_t st);
// conv_sparse.cu
bool conv_sparse_supported(int dtype, int kv, int K, int N);
int conv_gather_sparse(const void* rows, int dtype, int64_t n_rows, const void* weight, const int* nbr, int64_t n_out,
                       int kv, int K, int N, int flip_k, const float* scale, const float* bias, int relu, void* out,
                       int out_dtype, int* status, cudaStream_t st);

bool conv_wgrad_pairs_supported(int dtype, int kv, int K, int N);
int conv_wgrad_pairs(const void* rows, const void* dout, int dtype, int64_t n_rows, const int* nbr, int64_t n_out,
                     int kv, int K, int N, float* dw, int* status, cudaStream_t st);

// conv_wgrad_tc.cu
bool conv_wgrad_tc_supported(int dtype, int kv, int K, int N);
int conv_wgrad_tc(const void* rows, const void* dout, int dtype, int64_t n_rows, const int* nbr, int64_t n_out, int kv,
                  int K, int N, float* dw, int* status, cudaStream_t st);

}  // namespace sph

using namespace sph;

extern "C" const char* sph_last_error(void) { return g_err; }
extern "C" int sph_version(void) { return 100; }
extern "C" int64_t sph_kernel_launches(void) { return (int64_t)g_launches.load(std::memory_order_relaxed); }

extern "C" int64_t sph_packed_weight_bytes(int dtype, int32_t kv, int32_t k_ch, int32_t n_ch) {
  if (!conv_tc_supported(dtype, kv, k_ch, n_ch)) return 0;
  return packed_weight_bytes(dtype, kv, k_ch, n_ch);
}

extern "C" int sph_pack_weight(const void* d_weight, int dtype, int32_t kv, int32_t k_ch, int32_t n_ch,
                               void* d_packed, void* stream) {
  SPH_CHECK_ARG(d_weight && d_packed, "null pointer");
  return pack_weight(d_weight, dtype, kv, k_ch, n_ch, d_packed, (cudaStream_t)stream);
}

extern "C" int sph_conv_uses_tensor_cores(int dtype, int32_t k_ch, int32_t n_ch) {
  return conv_tc_supported(dtype, 27, k_ch, n_ch) ? 1 : 0;
}

extern "C" int sph_conv_uses_pair_kernel(int dtype, int32_t k_ch, int32_t n_ch) {
  return (!conv_tc_supported(dtype, 27, k_ch, n_ch) && conv_sparse_supported(dtype, 27, k_ch, n_ch)) ? 1 : 0;
}

extern "C" int sph_conv_wgrad_kernel(int dtype, int32_t k_ch, int32_t n_ch) {
  if (conv_wgrad_tc_supported(dtype, 27, k_ch, n_ch)) return 1;
  return conv_wgrad_pairs_supported(dtype, 27, k_ch, n_ch) ? 2 : 0;
}

static bool out_dtype_ok(int dtype, int out_dtype) {
  if (out_dtype < SPH_F32 || out_dtype > SPH_I8) return false;
  if (out_dtype == SPH_I8 && dtype != SPH_I8) return false;
  return true;
}

extern "C" int sph_conv_gather(const void* d_rows, int dtype, int64_t n_rows, const void* d_weight,
                               const void* d_packed, const int32_t* d_nbr, int64_t n_out, int32_t kv, int32_t k_ch,
                               int32_t n_ch, int flip_k, const float* d_scale, const float* d_bias, int relu,
                               void* d_out, int out_dtype, int32_t* d_status, void* stream) {
  SPH_CHECK_ARG(n_rows >= 0 && n_out >= 0 && kv > 0 && k_ch > 0 && n_ch > 0, "bad sizes");
  SPH_CHECK_ARG(dtype >= SPH_F32 && dtype <= SPH_I8, "unknown dtype");
  SPH_CHECK_ARG(out_dtype_ok(dtype, out_dtype), "unsupported output dtype for this input dtype");
  if (n_out == 0) return SPH_OK;
  SPH_CHECK_ARG(d_nbr && d_out && (d_weight || d_packed), "null pointer");
  SPH_CHECK_ARG(n_rows == 0 || d_rows, "null rows");
  SPH_CHECK_ARG(n_rows < 0x7fffffffLL && n_out < 0x7fffffffLL, "row ids are 32-bit");
  cudaStream_t st = (cudaStream_t)stream;
  // 64-byte rows: the form with the output row on the TMEM lane (absent neighbours masked, not copied) is the faster
  // of the two; wider rows are dense deep layers, where the transposed form issues half as many instructions
  if (d_packed && k_ch * dtype_bytes(dtype) == 64 && conv_tc_rows_supported(dtype, kv, k_ch, n_ch)) {
    return conv_gather_tc_rows(d_rows, dtype, n_rows, d_packed, d_nbr, n_out, kv, k_ch, n_ch, flip_k, d_scale, d_bias,
                               relu, d_out, out_dtype, d_status, st);
  }
  if (d_packed && conv_tc_supported(dtype, kv, k_ch, n_ch)) {
    return conv_gather_tc(d_rows, dtype, n_rows, d_packed, d_nbr, n_out, kv, k_ch, n_ch, flip_k, d_scale, d_bias,
                          relu, d_out, out_dtype, d_status, st);
  }
  SPH_CHECK_ARG(d_weight, "the CUDA-core kernels need the unpacked weight");
  // narrow rows the tensor-core kernels do not take (the first layer of an encoder: 4 or 8 channels in, a sparse level;
  // int8 rows of up to 16 channels) and small fp32 layers: the pair-compacting kernel (faster than the row-walking one from 1 to 22 neighbours per row)
  if (conv_sparse_supported(dtype, kv, k_ch, n_ch) &&
      ((((uintptr_t)d_rows | (uintptr_t)d_weight | (uintptr_t)d_out) & 15u) == 0)) {
    return conv_gather_sparse(d_rows, dtype, n_rows, d_weight, d_nbr, n_out, kv, k_ch, n_ch, flip_k, d_scale, d_bias,
                              relu, d_out, out_dtype, d_status, st);
  }
  return conv_gather_generic(d_rows, dtype, n_rows, d_weight, d_nbr, n_out, kv, k_ch, n_ch, flip_k, d_scale, d_bias,
                             relu, d_out, out_dtype, d_status, st);
}

extern "C" int sph_conv_wgrad(const void* d_rows, const void* d_dout, int dtype, int64_t n_rows,
                              const int32_t* d_nbr, int64_t n_out, int32_t kv, int32_t k_ch, int32_t n_ch,
                              float* d_dweight, int zero_init, int32_t* d_status, void* stream) {
  SPH_CHECK_ARG(n_rows >= 0 && n_out >= 0 && kv > 0 && k_ch > 0 && n_ch > 0, "bad sizes");
  SPH_CHECK_ARG(d_dweight, "null gradient buffer");
  cudaStream_t st = (cudaStream_t)stream;
  if (zero_init) SPH_CUDA(cudaMemsetAsync(d_dweight, 0, (size_t)kv * k_ch * n_ch * sizeof(float), st));
  if (n_out == 0 || n_rows == 0) return SPH_OK;
  SPH_CHECK_ARG(d_rows && d_dout && d_nbr, "null pointer");
  if (conv_wgrad_tc_supported(dtype, kv, k_ch, n_ch))
    return conv_wgrad_tc(d_rows, d_dout, dtype, n_rows, d_nbr, n_out, kv, k_ch, n_ch, d_dweight, d_status, st);
  // narrow rows the tensor-core kernel does not take and small fp32 layers: the pair-compacting walk
  if (conv_wgrad_pairs_supported(dtype, kv, k_ch, n_ch) && ((((uintptr_t)d_rows | (uintptr_t)d_dout) & 15u) == 0))
    return conv_wgrad_pairs(d_rows, d_dout, dtype, n_rows, d_nbr, n_out, kv, k_ch, n_ch, d_dweight, d_status, st);
  return conv_wgrad_generic(d_rows, d_dout, dtype, n_rows, d_nbr, n_out, kv, k_ch, n_ch, d_dweight, d_status, st);
}
