// Row kernels of a 32-bit residual stream whose sub-layers are normed on BOTH sides
// (x <- x + norm_b(f(norm_a(x)))), with norms that may subtract the mean:
//
//   norm_add_norm   stream[t] += mult * w * n(a[t])            (a absent: nothing is added)
//                   stream[t] += extra_rows[t]; stream[t] += extra_vec     (each optional, in this order)
//                   out[t] = round(w2 * n2(stream[t]))          (optional: the norm that reads the stream next)
//   norm_rows       out[r] = round(w * n(stream[rows[r]]))      (gathered rows; `rows` null: all in order)
//   xielu           out = round(act(in)), act(z) = softplus(p) z^2 + z / 2 for z > 0,
//                                          (1/2 + softplus(q)) (e^z - 1 - z) + z / 2 otherwise
//
// n(v) = v / sqrt(mean(v^2) + eps), or with `center` = 1 (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps): the
// variance is the mean of the squared deviations, formed in a second pass over the row, which waits in shared
// memory.  `center` = 2 for the added operand: n(v) = v, so stream[t] += mult * w * a[t] (a scale per channel on a
// sub-layer's output; w null: no scale), the arrangement of a pre-norm layer on a 32-bit stream.  Sums, means and the stream are 32-bit; one rounding at each store.  One block per row.
#include "common.cuh"

#define SN_MAX_SMEM (160 * 1024)

// (sum of v, then sum of squared deviations) or (sum of squares): returns the factor 1 / sqrt(.. + eps) and
// leaves the mean (0 without `center`) in *mean_out.
__device__ __forceinline__ float row_rstd(const float* row, int cols, bool center, float eps, float* scratch,
                                          float* mean_out) {
  float mean = 0.f;
  if (center) {
    float acc = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) acc += row[c];
    mean = block_sum(acc, scratch) / (float)cols;
  }
  float acc = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float d = row[c] - mean;
    acc += d * d;
  }
  *mean_out = mean;
  return 1.f / sqrtf(block_sum(acc, scratch) / (float)cols + eps);
}

template <typename TA, typename TO>
__global__ void norm_add_norm_kernel(const TA* __restrict__ a, float* __restrict__ stream,
                                     const float* __restrict__ w, int cols, float eps, float mult, int center,
                                     const float* __restrict__ extra_rows, const float* __restrict__ extra_vec,
                                     const float* __restrict__ w2, float eps2, int center2, TO* __restrict__ out) {
  extern __shared__ float sn_smem[];  // [cols] the operand's row, then [cols] the stream's row
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const long long base = (long long)blockIdx.x * cols;
  float* row_a = sn_smem;
  float* row_s = sn_smem + cols;
  float rstd = 0.f, mean = 0.f;
  if (a != nullptr) {
    for (int c = threadIdx.x; c < cols; c += blockDim.x) row_a[c] = to_f32(a[base + c]);
    __syncthreads();
    rstd = 1.f;
    if (center != 2) rstd = row_rstd(row_a, cols, center != 0, eps, scratch, &mean);
  }
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float s = stream[base + c];
    if (a != nullptr) s += mult * ((row_a[c] - mean) * rstd * (w != nullptr ? w[c] : 1.f));
    if (extra_rows != nullptr) s += extra_rows[base + c];
    if (extra_vec != nullptr) s += extra_vec[c];
    stream[base + c] = s;
    row_s[c] = s;
  }
  if (out == nullptr) return;
  __syncthreads();
  float mean2;
  const float rstd2 = row_rstd(row_s, cols, center2 != 0, eps2, scratch, &mean2);
  for (int c = threadIdx.x; c < cols; c += blockDim.x)
    out[base + c] = from_f32<TO>((row_s[c] - mean2) * rstd2 * w2[c]);
}

template <typename TO>
__global__ void norm_rows_kernel(const float* __restrict__ stream, const int* __restrict__ rows,
                                 const float* __restrict__ w, TO* __restrict__ out, int cols, int src_rows, float eps,
                                 int center, int* status) {
  extern __shared__ float sn_smem[];
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  int r = rows != nullptr ? rows[blockIdx.x] : (int)blockIdx.x;
  const bool bad = r < 0 || r >= src_rows;
  if (bad) {
    if (threadIdx.x == 0) ullm_report(status, ULLM_STATUS_ROW, blockIdx.x, r);
    r = 0;
  }
  const float* s = stream + (long long)r * cols;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) sn_smem[c] = s[c];
  __syncthreads();
  float mean;
  const float rstd = row_rstd(sn_smem, cols, center != 0, eps, scratch, &mean);
  for (int c = threadIdx.x; c < cols; c += blockDim.x)
    out[(long long)blockIdx.x * cols + c] = from_f32<TO>(bad ? 0.f : (sn_smem[c] - mean) * rstd * w[c]);
}

__device__ __forceinline__ float softplus_f32(float v) { return log1pf(expf(-fabsf(v))) + fmaxf(v, 0.f); }

template <typename T>
__global__ void xielu_kernel(const T* __restrict__ in, T* __restrict__ out, long long n,
                             const float* __restrict__ pq) {
  pdl_launch_dependents();
  pdl_wait();
  const float ap = softplus_f32(pq[0]), aq = 0.5f + softplus_f32(pq[1]);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float z = to_f32(in[i]);
    const float y = z > 0.f ? ap * z * z + 0.5f * z : aq * (expm1f(z) - z) + 0.5f * z;
    out[i] = from_f32<T>(y);
  }
}

static inline int sn_threads(int cols) {
  int threads = 32;
  while (threads < 512 && threads * 4 < cols) threads <<= 1;
  return threads;
}

template <typename K>
static int sn_allow_smem(K kernel, size_t smem) {
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    cudaGetLastError();
    return ULLM_ERR_UNSUPPORTED;
  }
  return ULLM_OK;
}

template <typename TA, typename TO>
static int norm_add_norm_launch(const void* a, float* stream, const float* w, int rows, int cols, float eps,
                                float mult, int center, const float* extra_rows, const float* extra_vec,
                                const float* w2, float eps2, int center2, void* out, cudaStream_t st) {
  const size_t smem = 2 * (size_t)cols * sizeof(float);
  if (smem > SN_MAX_SMEM) return ULLM_ERR_UNSUPPORTED;
  const int rc = sn_allow_smem(norm_add_norm_kernel<TA, TO>, smem);
  if (rc != ULLM_OK) return rc;
  return ullm_launch_kernel(norm_add_norm_kernel<TA, TO>, dim3(rows), dim3(sn_threads(cols)), smem, st,
                            (const TA*)a, stream, w, cols, eps, mult, center, extra_rows, extra_vec, w2, eps2,
                            center2, (TO*)out);
}

// `a_dtype`: dtype of `a` (the engine's, or 32-bit for a sub-layer that leaves 32-bit rows); `out_dtype`: of `out`.
// `a` null: nothing is normed and added (then `w` is unused); `out` null: no next norm.
extern "C" int ullm_norm_add_norm(int a_dtype, const void* a, float* stream, const float* w, int rows, int cols,
                                  float eps, float mult, int center, const float* extra_rows,
                                  const float* extra_vec, const float* w2, float eps2, int center2, int out_dtype,
                                  void* out, void* stream_handle) {
  cudaStream_t st = (cudaStream_t)stream_handle;
  if (rows < 0 || cols <= 0) return ULLM_ERR_BAD_SIZE;
  if ((a != nullptr && w == nullptr && center != 2) || (out != nullptr && w2 == nullptr)) return ULLM_ERR_BAD_SIZE;
  if (center < 0 || center > 2 || center2 < 0 || center2 > 1) return ULLM_ERR_BAD_SIZE;
  if (rows == 0) return ULLM_OK;
#define SN_GO(TA, TO)                                                                                              \
  return norm_add_norm_launch<TA, TO>(a, stream, w, rows, cols, eps, mult, center, extra_rows, extra_vec, w2, eps2, \
                                      center2, out, st)
#define SN_OUT(TA)                                         \
  if (out_dtype == ULLM_DTYPE_F32) SN_GO(TA, float);       \
  if (out_dtype == ULLM_DTYPE_BF16) SN_GO(TA, __nv_bfloat16); \
  if (out_dtype == ULLM_DTYPE_F16) SN_GO(TA, __half);      \
  return ULLM_ERR_BAD_DTYPE
  if (a_dtype == ULLM_DTYPE_F32) { SN_OUT(float); }
  if (a_dtype == ULLM_DTYPE_BF16) { SN_OUT(__nv_bfloat16); }
  if (a_dtype == ULLM_DTYPE_F16) { SN_OUT(__half); }
#undef SN_OUT
#undef SN_GO
  return ULLM_ERR_BAD_DTYPE;
}

template <typename TO>
static int norm_rows_launch(const float* stream, const int* rows, const float* w, void* out, int count, int cols,
                            int src_rows, float eps, int center, int* status, cudaStream_t st) {
  const size_t smem = (size_t)cols * sizeof(float);
  if (smem > SN_MAX_SMEM) return ULLM_ERR_UNSUPPORTED;
  const int rc = sn_allow_smem(norm_rows_kernel<TO>, smem);
  if (rc != ULLM_OK) return rc;
  return ullm_launch_kernel(norm_rows_kernel<TO>, dim3(count), dim3(sn_threads(cols)), smem, st, stream, rows, w,
                            (TO*)out, cols, src_rows, eps, center, status);
}

extern "C" int ullm_norm_rows(int dtype, const float* stream, const int* rows, const float* w, void* out, int count,
                              int cols, int src_rows, float eps, int center, int* status, void* stream_handle) {
  cudaStream_t st = (cudaStream_t)stream_handle;
  if (count < 0 || cols <= 0 || src_rows < 0) return ULLM_ERR_BAD_SIZE;
  if (count == 0) return ULLM_OK;
  if (dtype == ULLM_DTYPE_F32)
    return norm_rows_launch<float>(stream, rows, w, out, count, cols, src_rows, eps, center, status, st);
  if (dtype == ULLM_DTYPE_BF16)
    return norm_rows_launch<__nv_bfloat16>(stream, rows, w, out, count, cols, src_rows, eps, center, status, st);
  if (dtype == ULLM_DTYPE_F16)
    return norm_rows_launch<__half>(stream, rows, w, out, count, cols, src_rows, eps, center, status, st);
  return ULLM_ERR_BAD_DTYPE;
}

// out = act(in) element by element; `pq`: the activation's two numbers (32-bit, on the device).
extern "C" int ullm_xielu(int dtype, const void* in, void* out, long long n, const float* pq, void* stream_handle) {
  cudaStream_t st = (cudaStream_t)stream_handle;
  if (n < 0 || pq == nullptr) return ULLM_ERR_BAD_SIZE;
  if (n == 0) return ULLM_OK;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  const dim3 grid((int)blocks), block(256);
  if (dtype == ULLM_DTYPE_F32)
    return ullm_launch_kernel(xielu_kernel<float>, grid, block, 0, st, (const float*)in, (float*)out, n, pq);
  if (dtype == ULLM_DTYPE_BF16)
    return ullm_launch_kernel(xielu_kernel<__nv_bfloat16>, grid, block, 0, st, (const __nv_bfloat16*)in,
                              (__nv_bfloat16*)out, n, pq);
  if (dtype == ULLM_DTYPE_F16)
    return ullm_launch_kernel(xielu_kernel<__half>, grid, block, 0, st, (const __half*)in, (__half*)out, n, pq);
  return ULLM_ERR_BAD_DTYPE;
}
