// A residual stream kept in 32-bit whatever the engine's dtype, for
// arrangements that norm a sub-layer's OUTPUT and add it to the stream:
//
//   embed_scaled      stream[t] = table[id[t]] * scale (+ sinusoid of the position), copy[t] = round(stream[t])
//   norm_scale_add    stream[t] += mult * w * a[t] / sqrt(mean(a[t]^2) + eps),       copy[t] = round(stream[t])
//   norm_scale_add_norm   the same, and out[t] = the NEXT norm of the updated stream[t]
//   rmsnorm_rows_f32  out[r] = round(w * s / sqrt(mean(s^2) + eps)), s = stream[rows[r]]
//   cast_rows_f32     copy = round(stream)
//   concat_rows_f32   out[t] = round([a[t] | b[t]]): two 32-bit row sets side by side as one product's operand
//   sigmoid_gate      a[t] *= sigmoid(g[t]), element by element (g with a row stride of its own)
//   gated_add_f32     stream[t] += sigmoid(g1[t] + b1) * a[t] (+ sigmoid(g2[t] + b2) * f[t]),       copy[t] = round(stream[t])
//   side_gate_mul     out[t] = gelu_tanh(s[t]) * table[id[t]][offset .. offset + cols)
//   softcap_f32       x = cap * tanh(x / cap), in place
//
// `copy` is the stream rounded to the engine's dtype, the operand of the next
// sub-layer's matrix products; with a 32-bit engine it is not needed (null).
// Sums, norms, angles and the sinusoids are 32-bit; one rounding at each store.
#include "common.cuh"

// Position term: column c of position p is sin(p f_i) for even c and cos(p f_i) for odd c, i = c / 2, with
// f_i = base^(-2 i / width) read from a 32-bit table the host built in 64-bit.  The angle is the 32-bit
// product; sinf / cosf are the accurate forms (full range reduction).
template <typename T, typename TAB>
__global__ void embed_scaled_kernel(const int* __restrict__ ids, const TAB* __restrict__ table,
                                    float* __restrict__ stream, T* __restrict__ copy, int hidden, int vocab,
                                    float scale, const float* __restrict__ inv_freq,
                                    const int* __restrict__ positions, const int* __restrict__ last_tokens,
                                    const int* __restrict__ token_req, const int* __restrict__ req_slots,
                                    int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 && last_tokens != nullptr) {
    const int b = token_req[t];
    id = b >= 0 ? last_tokens[req_slots[b]] : 0;
  }
  const bool bad = id < 0 || id >= vocab;
  if (bad && threadIdx.x == 0) ullm_report(status, ULLM_STATUS_TOKEN_ID, t, id);
  const TAB* row = table + (long long)(bad ? 0 : id) * hidden;
  const float p = inv_freq != nullptr ? (float)positions[t] : 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = bad ? 0.f : to_f32(row[c]) * scale;
    if (inv_freq != nullptr) {
      const float ang = p * inv_freq[c >> 1];
      v += (c & 1) ? cosf(ang) : sinf(ang);
    }
    stream[(long long)t * hidden + c] = v;
    if (copy != nullptr) copy[(long long)t * hidden + c] = from_f32<T>(v);
  }
}

template <typename T>
__global__ void norm_scale_add_kernel(const T* __restrict__ a, float* __restrict__ stream,
                                      const float* __restrict__ w, T* __restrict__ copy, int cols, float eps,
                                      float mult) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const long long base = (long long)blockIdx.x * cols;
  float acc = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = to_f32(a[base + c]);
    acc += v * v;
  }
  const float total = block_sum(acc, scratch);
  const float rstd = 1.f / sqrtf(total / (float)cols + eps);
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float s = stream[base + c] + mult * (to_f32(a[base + c]) * rstd * w[c]);
    stream[base + c] = s;
    if (copy != nullptr) copy[base + c] = from_f32<T>(s);
  }
}

// The same, and in the same pass the NEXT norm of the updated stream: out[t] = round(w2 * s / sqrt(mean(s^2) + eps2))
// for s = the stream's new row, which waits in shared memory (`cols` floats) between the two sums: the stream is
// neither written and read again nor normed by a kernel of its own.
template <typename T>
__global__ void norm_scale_add_norm_kernel(const T* __restrict__ a, float* __restrict__ stream,
                                           const float* __restrict__ w, int cols, float eps, float mult,
                                           const float* __restrict__ w2, float eps2, T* __restrict__ out) {
  extern __shared__ float row_s[];
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const long long base = (long long)blockIdx.x * cols;
  float acc = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = to_f32(a[base + c]);
    acc += v * v;
  }
  const float rstd = 1.f / sqrtf(block_sum(acc, scratch) / (float)cols + eps);
  float acc2 = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float s = stream[base + c] + mult * (to_f32(a[base + c]) * rstd * w[c]);
    stream[base + c] = s;
    row_s[c] = s;
    acc2 += s * s;
  }
  const float rstd2 = 1.f / sqrtf(block_sum(acc2, scratch) / (float)cols + eps2);
  for (int c = threadIdx.x; c < cols; c += blockDim.x) out[base + c] = from_f32<T>(row_s[c] * rstd2 * w2[c]);
}

template <typename T>
__global__ void rmsnorm_rows_f32_kernel(const float* __restrict__ stream, const int* __restrict__ rows,
                                        const float* __restrict__ w, T* __restrict__ out, int cols, int src_rows,
                                        float eps, int* status) {
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
  float acc = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) acc += s[c] * s[c];
  const float total = block_sum(acc, scratch);
  const float rstd = 1.f / sqrtf(total / (float)cols + eps);
  for (int c = threadIdx.x; c < cols; c += blockDim.x)
    out[(long long)blockIdx.x * cols + c] = from_f32<T>(bad ? 0.f : s[c] * rstd * w[c]);
}

template <typename T>
__global__ void cast_rows_f32_kernel(const float* __restrict__ in, T* __restrict__ out, long long n) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = from_f32<T>(in[i]);
}

template <typename T>
__global__ void concat_rows_f32_kernel(const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ out,
                                       int cols_a, int cols_b) {
  pdl_launch_dependents();
  pdl_wait();
  const long long t = blockIdx.x;
  T* o = out + t * (cols_a + cols_b);
  for (int c = threadIdx.x; c < cols_a; c += blockDim.x) o[c] = from_f32<T>(a[t * cols_a + c]);
  for (int c = threadIdx.x; c < cols_b; c += blockDim.x) o[cols_a + c] = from_f32<T>(b[t * cols_b + c]);
}

template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ a, const T* __restrict__ g, long long g_stride, int cols) {
  pdl_launch_dependents();
  pdl_wait();
  const long long t = blockIdx.x;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float z = to_f32(g[t * g_stride + c]);
    a[t * cols + c] = from_f32<T>(to_f32(a[t * cols + c]) / (1.f + expf(-z)));
  }
}

// Two sub-layers that read the same normed rows and are added to the stream together, each through a gate:
// stream += sigmoid(g1 + b1) * a + sigmoid(g2 + b2) * f.  g1 | g2 are the columns of ONE 32-bit product
// (row stride `g_stride`); f, g2 and b2 are absent for a layer without the second sub-layer.
template <typename T>
__global__ void gated_add_f32_kernel(const T* __restrict__ a, const T* __restrict__ f, const float* __restrict__ g,
                                     long long g_stride, const float* __restrict__ b1, const float* __restrict__ b2,
                                     float* __restrict__ stream, T* __restrict__ copy, int cols) {
  pdl_launch_dependents();
  pdl_wait();
  const long long base = (long long)blockIdx.x * cols;
  const float* gr = g + (long long)blockIdx.x * g_stride;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float y = to_f32(a[base + c]) / (1.f + expf(-(gr[c] + b1[c])));
    if (f != nullptr) y += to_f32(f[base + c]) / (1.f + expf(-(gr[cols + c] + b2[c])));
    const float s = stream[base + c] + y;
    stream[base + c] = s;
    if (copy != nullptr) copy[base + c] = from_f32<T>(s);
  }
}

// out[t][c] = gelu_tanh(s[t][c]) * table[id[t]][offset + c]: a per-token input (a second embedding table, of which
// a layer reads `cols` columns from `offset` on) gated by a projection of the stream.  An id of -1 is the token
// the request sampled last, as in the embedding kernels.
template <typename T>
__global__ void side_gate_mul_kernel(const T* __restrict__ s, const int* __restrict__ ids, const T* __restrict__ table,
                                     long long table_stride, int offset, T* __restrict__ out, int cols, int vocab,
                                     const int* __restrict__ last_tokens, const int* __restrict__ token_req,
                                     const int* __restrict__ req_slots, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 && last_tokens != nullptr) {
    const int b = token_req[t];
    id = b >= 0 ? last_tokens[req_slots[b]] : 0;
  }
  const bool bad = id < 0 || id >= vocab;
  if (bad && threadIdx.x == 0) ullm_report(status, ULLM_STATUS_TOKEN_ID, t, id);
  const T* row = table + (long long)(bad ? 0 : id) * table_stride + offset;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = act_gelu_tanh(to_f32(s[(long long)t * cols + c])) * (bad ? 0.f : to_f32(row[c]));
    out[(long long)t * cols + c] = from_f32<T>(v);
  }
}

__global__ void softcap_f32_kernel(float* __restrict__ x, long long n, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  const float inv = 1.f / cap;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    x[i] = cap * tanhf(x[i] * inv);
}

static inline int row_threads(int cols) {
  int threads = 32;
  while (threads < 512 && threads * 4 < cols) threads <<= 1;
  return threads;
}

template <typename T, typename TAB>
static int embed_scaled_launch(const int* ids, const void* table, float* stream, void* copy, int tokens, int hidden,
                               int vocab, float scale, const float* inv_freq, const int* positions,
                               const int* last_tokens, const int* token_req, const int* req_slots, int* status,
                               cudaStream_t st) {
  return ullm_launch_kernel(embed_scaled_kernel<T, TAB>, dim3(tokens), dim3(row_threads(hidden)), 0, st, ids,
                            (const TAB*)table, stream, (T*)copy, hidden, vocab, scale, inv_freq, positions,
                            last_tokens, token_req, req_slots, status);
}

// `dtype`: the engine's dtype = the table's and the copy's.  `copy` may be null.
extern "C" int ullm_embed_scaled(int dtype, const int* ids, const void* table, float* stream, void* copy, int tokens,
                                 int hidden, int vocab, float scale, const float* inv_freq, const int* positions,
                                 const int* last_tokens, const int* token_req, const int* req_slots, int* status,
                                 void* stream_handle) {
  cudaStream_t st = (cudaStream_t)stream_handle;
  if (tokens < 0 || hidden <= 0 || vocab <= 0) return ULLM_ERR_BAD_SIZE;
  if (inv_freq != nullptr && positions == nullptr) return ULLM_ERR_BAD_SIZE;
  if (last_tokens != nullptr && (token_req == nullptr || req_slots == nullptr)) return ULLM_ERR_BAD_SIZE;
  if (tokens == 0) return ULLM_OK;
  if (dtype == ULLM_DTYPE_F32)
    return embed_scaled_launch<float, float>(ids, table, stream, copy, tokens, hidden, vocab, scale, inv_freq,
                                             positions, last_tokens, token_req, req_slots, status, st);
  if (dtype == ULLM_DTYPE_BF16)
    return embed_scaled_launch<__nv_bfloat16, __nv_bfloat16>(ids, table, stream, copy, tokens, hidden, vocab, scale,
                                                             inv_freq, positions, last_tokens, token_req, req_slots,
                                                             status, st);
  if (dtype == ULLM_DTYPE_F16)
    return embed_scaled_launch<__half, __half>(ids, table, stream, copy, tokens, hidden, vocab, scale, inv_freq,
                                               positions, last_tokens, token_req, req_slots, status, st);
  return ULLM_ERR_BAD_DTYPE;
}

extern "C" int ullm_norm_scale_add(int dtype, const void* a, float* stream, const float* w, void* copy, int rows,
                                   int cols, float eps, float mult, void* stream_handle) {
  cudaStream_t st = (cudaStream_t)stream_handle;
  if (rows < 0 || cols <= 0) return ULLM_ERR_BAD_SIZE;
  if (rows == 0) return ULLM_OK;
  const dim3 grid(rows), block(row_threads(cols));
  if (dtype == ULLM_DTYPE_F32)
    return ullm_launch_kernel(norm_scale_add_kernel<float>, grid, block, 0, st, (const float*)a, stream, w,
                              (float*)copy, cols, eps, mult);
  if (dtype == ULLM_DTYPE_BF16)
    return ullm_launch_kernel(norm_scale_add_kernel<__nv_bfloat16>, grid, block, 0, st, (const __nv_bfloat16*)a,
                              stream, w, (__nv_bfloat16*)copy, cols, eps, mult);
  if (dtype == ULLM_DTYPE_F16)
    return ullm_launch_kernel(norm_scale_add_kernel<__half>, grid, block, 0, st, (const __half*)a, stream, w,
                              (__half*)copy, cols, eps, mult);
  return ULLM_ERR_BAD_DTYPE;
}

// stream += mult * w * a / rms(a), and out = the next norm (w2, eps2) of the updated stream, in one kernel.
extern "C" int ullm_norm_scale_add_norm(int dtype, const void* a, float* stream, const float* w, int rows, int cols,
                                        float eps, float mult, const float* w2, float eps2, void* out,
                                        void* stream_handle) {
  cudaStream_t st = (cudaStream_t)stream_handle;
  if (rows < 0 || cols <= 0) return ULLM_ERR_BAD_SIZE;
  if ((size_t)cols * sizeof(float) > 40 * 1024) return ULLM_ERR_UNSUPPORTED;
  if (rows == 0) return ULLM_OK;
  const dim3 grid(rows), block(row_threads(cols));
  const size_t smem = (size_t)cols * sizeof(float);
  if (dtype == ULLM_DTYPE_F32)
    return ullm_launch_kernel(norm_scale_add_norm_kernel<float>, grid, block, smem, st, (const float*)a, stream, w,
                              cols, eps, mult, w2, eps2, (float*)out);
  if (dtype == ULLM_DTYPE_BF16)
    return ullm_launch_kernel(norm_scale_add_norm_kernel<__nv_bfloat16>, grid, block, smem, st,
                              (const __nv_bfloat16*)a, stream, w, cols, eps, mult, w2, eps2, (__nv_bfloat16*)out);
  if (dtype == ULLM_DTYPE_F16)
    return ullm_launch_kernel(norm_scale_add_norm_kernel<__half>, grid, block, smem, st, (const __half*)a, stream, w,
                              cols, eps, mult, w2, eps2, (__half*)out);
  return ULLM_ERR_BAD_DTYPE;
}

// `rows` may be null (row r of the output is row r of the stream).
extern "C" int ullm_rmsnorm_rows_f32(int dtype, const float* stream, const int* rows, const float* w, void* out,
                                     int count, int cols, int src_rows, float eps, int* status, void* stream_handle) {
  cudaStream_t st = (cudaStream_t)stream_handle;
  if (count < 0 || cols <= 0 || src_rows < 0) return ULLM_ERR_BAD_SIZE;
  if (count == 0) return ULLM_OK;
  const dim3 grid(count), block(row_threads(cols));
  if (dtype == ULLM_DTYPE_F32)
    return ullm_launch_kernel(rmsnorm_rows_f32_kernel<float>, grid, block, 0, st, stream, rows, w, (float*)out, cols,
                              src_rows, eps, status);
  if (dtype == ULLM_DTYPE_BF16)
    return ullm_launch_kernel(rmsnorm_rows_f32_kernel<__nv_bfloat16>, grid, block, 0, st, stream, rows, w,
                              (__nv_bfloat16*)out, cols, src_rows, eps, status);
  if (dtype == ULLM_DTYPE_F16)
    return ullm_launch_kernel(rmsnorm_rows_f32_kernel<__half>, grid, block, 0, st, stream, rows, w, (__half*)out,
                              cols, src_rows, eps, status);
  return ULLM_ERR_BAD_DTYPE;
}

extern "C" int ullm_cast_rows_f32(int dtype, const float* in, void* out, long long n, void* stream_handle) {
  cudaStream_t st = (cudaStream_t)stream_handle;
  if (n < 0) return ULLM_ERR_BAD_SIZE;
  if (n == 0) return ULLM_OK;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  const dim3 grid((int)blocks), block(256);
  if (dtype == ULLM_DTYPE_BF16)
    return ullm_launch_kernel(cast_rows_f32_kernel<__nv_bfloat16>, grid, block, 0, st, in, (__nv_bfloat16*)out, n);
  if (dtype == ULLM_DTYPE_F16)
    return ullm_launch_kernel(cast_rows_f32_kernel<__half>, grid, block, 0, st, in, (__half*)out, n);
  if (dtype == ULLM_DTYPE_F32)
    return ullm_launch_kernel(cast_rows_f32_kernel<float>, grid, block, 0, st, in, (float*)out, n);
  return ULLM_ERR_BAD_DTYPE;
}

// `f`, `b2` null: one gated sub-layer only (the product then has `cols` columns).
extern "C" int ullm_gated_add_f32(int dtype, const void* a, const void* f, const float* g, long long g_stride,
                                  const float* b1, const float* b2, float* stream, void* copy, int rows, int cols,
                                  void* stream_handle) {
  cudaStream_t st = (cudaStream_t)stream_handle;
  if (rows < 0 || cols <= 0 || g_stride < cols * (f != nullptr ? 2 : 1)) return ULLM_ERR_BAD_SIZE;
  if ((f != nullptr) != (b2 != nullptr)) return ULLM_ERR_BAD_SIZE;
  if (rows == 0) return ULLM_OK;
  const dim3 grid(rows), block(row_threads(cols));
  if (dtype == ULLM_DTYPE_F32)
    return ullm_launch_kernel(gated_add_f32_kernel<float>, grid, block, 0, st, (const float*)a, (const float*)f, g,
                              g_stride, b1, b2, stream, (float*)copy, cols);
  if (dtype == ULLM_DTYPE_BF16)
    return ullm_launch_kernel(gated_add_f32_kernel<__nv_bfloat16>, grid, block, 0, st, (const __nv_bfloat16*)a,
                              (const __nv_bfloat16*)f, g, g_stride, b1, b2, stream, (__nv_bfloat16*)copy, cols);
  if (dtype == ULLM_DTYPE_F16)
    return ullm_launch_kernel(gated_add_f32_kernel<__half>, grid, block, 0, st, (const __half*)a, (const __half*)f, g,
                              g_stride, b1, b2, stream, (__half*)copy, cols);
  return ULLM_ERR_BAD_DTYPE;
}

extern "C" int ullm_side_gate_mul(int dtype, const void* s, const int* ids, const void* table, long long table_stride,
                                  int offset, void* out, int tokens, int cols, int vocab, const int* last_tokens,
                                  const int* token_req, const int* req_slots, int* status, void* stream_handle) {
  cudaStream_t st = (cudaStream_t)stream_handle;
  if (tokens < 0 || cols <= 0 || vocab <= 0 || offset < 0 || offset + cols > table_stride) return ULLM_ERR_BAD_SIZE;
  if (last_tokens != nullptr && (token_req == nullptr || req_slots == nullptr)) return ULLM_ERR_BAD_SIZE;
  if (tokens == 0) return ULLM_OK;
  const dim3 grid(tokens), block(row_threads(cols));
  if (dtype == ULLM_DTYPE_F32)
    return ullm_launch_kernel(side_gate_mul_kernel<float>, grid, block, 0, st, (const float*)s, ids,
                              (const float*)table, table_stride, offset, (float*)out, cols, vocab, last_tokens,
                              token_req, req_slots, status);
  if (dtype == ULLM_DTYPE_BF16)
    return ullm_launch_kernel(side_gate_mul_kernel<__nv_bfloat16>, grid, block, 0, st, (const __nv_bfloat16*)s, ids,
                              (const __nv_bfloat16*)table, table_stride, offset, (__nv_bfloat16*)out, cols, vocab,
                              last_tokens, token_req, req_slots, status);
  if (dtype == ULLM_DTYPE_F16)
    return ullm_launch_kernel(side_gate_mul_kernel<__half>, grid, block, 0, st, (const __half*)s, ids,
                              (const __half*)table, table_stride, offset, (__half*)out, cols, vocab, last_tokens,
                              token_req, req_slots, status);
  return ULLM_ERR_BAD_DTYPE;
}

extern "C" int ullm_softcap_f32(float* x, long long n, float cap, void* stream_handle) {
  cudaStream_t st = (cudaStream_t)stream_handle;
  if (n < 0 || !(cap > 0.f)) return ULLM_ERR_BAD_SIZE;
  if (n == 0) return ULLM_OK;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return ullm_launch_kernel(softcap_f32_kernel, dim3((int)blocks), dim3(256), 0, st, x, n, cap);
}

extern "C" int ullm_concat_rows_f32(int dtype, const float* a, const float* b, void* out, int rows, int cols_a,
                                    int cols_b, void* stream_handle) {
  cudaStream_t st = (cudaStream_t)stream_handle;
  if (rows < 0 || cols_a <= 0 || cols_b <= 0) return ULLM_ERR_BAD_SIZE;
  if (rows == 0) return ULLM_OK;
  const dim3 grid(rows), block(row_threads(cols_a + cols_b));
  if (dtype == ULLM_DTYPE_F32)
    return ullm_launch_kernel(concat_rows_f32_kernel<float>, grid, block, 0, st, a, b, (float*)out, cols_a, cols_b);
  if (dtype == ULLM_DTYPE_BF16)
    return ullm_launch_kernel(concat_rows_f32_kernel<__nv_bfloat16>, grid, block, 0, st, a, b, (__nv_bfloat16*)out,
                              cols_a, cols_b);
  if (dtype == ULLM_DTYPE_F16)
    return ullm_launch_kernel(concat_rows_f32_kernel<__half>, grid, block, 0, st, a, b, (__half*)out, cols_a, cols_b);
  return ULLM_ERR_BAD_DTYPE;
}

extern "C" int ullm_sigmoid_gate(int dtype, void* a, const void* g, long long g_stride, int rows, int cols,
                                 void* stream_handle) {
  cudaStream_t st = (cudaStream_t)stream_handle;
  if (rows < 0 || cols <= 0 || g_stride < cols) return ULLM_ERR_BAD_SIZE;
  if (rows == 0) return ULLM_OK;
  const dim3 grid(rows), block(row_threads(cols));
  if (dtype == ULLM_DTYPE_F32)
    return ullm_launch_kernel(sigmoid_gate_kernel<float>, grid, block, 0, st, (float*)a, (const float*)g, g_stride, cols);
  if (dtype == ULLM_DTYPE_BF16)
    return ullm_launch_kernel(sigmoid_gate_kernel<__nv_bfloat16>, grid, block, 0, st, (__nv_bfloat16*)a,
                              (const __nv_bfloat16*)g, g_stride, cols);
  if (dtype == ULLM_DTYPE_F16)
    return ullm_launch_kernel(sigmoid_gate_kernel<__half>, grid, block, 0, st, (__half*)a, (const __half*)g, g_stride,
                              cols);
  return ULLM_ERR_BAD_DTYPE;
}
