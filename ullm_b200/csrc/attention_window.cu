// Windowed paged attention on the tensor cores for bfloat16 batches of any mix of prompt portions and single
// decoded tokens, with the options of the general kernel's `AttExtras` (csrc/attention_generic.cu): values that
// are the first `dv` elements of the key rows, distance slopes, pooled blocks behind the window, an output gate,
// an output scale and a row stride of the output.  Key rows of any size that is a multiple of 16 (the QK loop
// runs over a runtime count of 16-wide steps; the usual sizes are also compiled as constants), values up to 512.
//
// Flash-attention style, mma.sync m16n8k16 bf16 with 32-bit accumulation; scores, maxima, sums, the distance
// bias and the output accumulator are 32-bit.  A block owns 64 rows of one kv head for one request; rows are
// (token, query head of the group) pairs, so with G query heads per kv head it covers 64 / G tokens and one pass
// over the keys serves all heads that share them (latent attention: one kv head, G = all heads).  The block's
// warps form a grid of 4 row groups (16 rows each) x CW column groups: the warps of a row group split the
// 16-wide steps of Q K^T, add their partial scores through shared memory, form the same weights and apply them to
// their own DVW of the value columns, so the output accumulator of wide values is spread over CW warps' registers.
//
// Key tiles of 64, gathered from the pages by cp.async into a two-stage ring (rows padded by 16 bytes: with a
// row size that is a multiple of 32 bytes the eight rows of an ldmatrix fall into distinct banks); value pages
// of their own have one stage, awaited between the softmax and P V.  A block walks first the pooled entries its
// rows can see (entry b stands for positions bP .. bP + P - 1 and is seen by a row at position i when
// bP + P - 1 <= i - window), then the keys from the window's start of its first token to its last token.  All
// stretches share one online softmax.  For steps of few rows the tiles of a block are cut into runs (grid.y)
// whose unnormalised results a second kernel merges.  The only waits are cp.async groups and block barriers.
#include "common.cuh"

#define WIN_N 64
#define WIN_MAX_GROUP 64  // query heads per kv head: a token's heads lie in one block

struct WinArgs {
  const __nv_bfloat16* q;
  long long q_stride;
  __nv_bfloat16* out;
  long long out_stride;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;  // null: a head's values are the first dv elements of its key row
  const int* block_table;
  int max_pages;
  long long num_pages;
  const int* req_slots;
  const int* cu_q;
  const int* kv_len;
  int num_requests, num_q, num_kv, dk, dv, page_size, window;
  float scale_log2;
  const float* slopes;
  int pool;
  const __nv_bfloat16* pk;
  const __nv_bfloat16* pv;
  const int* p_block_table;
  int p_max_pages;
  long long p_num_pages;
  const __nv_bfloat16* gate;
  long long gate_stride;
  float out_scale;
  int* status;
  // nsplit > 1: the block's key tiles are cut into nsplit runs, one block each (grid.y); a block leaves its
  // unnormalised 32-bit accumulator, maximum (in units of log2) and sum in `parts`
  // [token x head][nsplit][dv + 2], and `window_merge_kernel` forms the output rows
  int nsplit;
  float* parts;
  int ksplit;  // the column groups of a row group share the steps of Q K^T (needs the exchange buffer)
};

__device__ __forceinline__ void win_cp_async_16(void* smem, const void* gmem, bool pred) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int n = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void win_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void win_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void win_ldsm4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(s));
}
__device__ __forceinline__ void win_ldsm4t(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(s));
}
__device__ __forceinline__ void win_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x, one instruction of the special-function unit; 2^(-inf) = 0
__device__ __forceinline__ float win_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned win_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// values up to 128 wide: one column group; up to 256: two; up to 384: three of 128; up to 512: two of 256.  Four row groups (with eight, 256 threads of about 170
// registers leave one block per SM; four leave three)
static inline int win_row_groups(int dv) { return 4; }
static inline int win_col_groups(int dv) { return dv <= 128 ? 1 : (dv > 256 && dv <= 384 ? 3 : 2); }
static inline long long win_smem_bytes(int dk, int dv, bool v_own) {
  const long long qs = dk * 2 + 16, vs = dv * 2 + 16;
  return 16LL * win_row_groups(dv) * qs + 2LL * WIN_N * qs + (v_own ? 1LL * WIN_N * vs : 0) + 2LL * WIN_N * 8;
}
// the partial scores that the column groups of a row group exchange: [row group][column group][32 registers][lane]
static inline long long win_exchange_bytes(int dv) {
  return win_col_groups(dv) > 1 ? 4096LL * win_row_groups(dv) * win_col_groups(dv) : 0;
}

// DKT > 0: the key rows are DKT wide and the values DVW x CW, known to the compiler (strides, piece counts and the
// steps of Q K^T become constants and the loops unroll); DKT = 0: both are read from the arguments.
template <int DVW, int CW, int RW, int DKT>
__global__ void __launch_bounds__(RW * CW * 32, CW == 1 ? 3 : 1) window_attention_kernel(const WinArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  pdl_launch_dependents();
  pdl_wait();
  constexpr int NT_S = WIN_N / 8, NT_O = DVW / 8, THREADS = RW * CW * 32, WIN_M = RW * 16;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rw = warp % RW, cw = warp / RW;
  const int dk = DKT > 0 ? DKT : a.dk, dv = DKT > 0 ? DVW * CW : a.dv, W = a.window, page_size = a.page_size;
  const bool v_own = a.v_cache != nullptr;
  const int qs = dk * 2 + 16;               // bytes between rows of the Q and K tiles
  const int vs = v_own ? dv * 2 + 16 : qs;  // ... of the tile the values are read from
  unsigned char* q_s = smem;
  unsigned char* k_s = q_s + WIN_M * qs;
  unsigned char* v_s = k_s + 2 * WIN_N * qs;
  long long* slot_s = reinterpret_cast<long long*>(v_s + (v_own ? WIN_N * vs : 0));
  float* exch_s = reinterpret_cast<float*>(slot_s + 2 * WIN_N);  // only with `ksplit`

  // consecutive blocks are the same token tile of all kv heads, the last tiles (most keys) first
  const int num_kv = a.num_kv;
  const int kh = (int)(blockIdx.x % num_kv);
  const int G = a.num_q / num_kv;
  const int tpt = WIN_M / G;  // tokens per block
  const int tile_id = (int)(gridDim.x / num_kv) - 1 - (int)(blockIdx.x / num_kv);
  int r = -1, first = 0, q_len = 0, q_begin = 0;
  {
    int running = 0;
    for (int i = 0; i < a.num_requests; ++i) {
      const int b = a.cu_q[i], n = a.cu_q[i + 1] - b;
      const int nt = (n + tpt - 1) / tpt;
      if (tile_id < running + nt) {
        r = i;
        first = (tile_id - running) * tpt;
        q_len = n;
        q_begin = b;
        break;
      }
      running += nt;
    }
  }
  if (r < 0) return;
  const int kvl = a.kv_len[r];
  const int ntok = min(tpt, q_len - first);
  const int rows_valid = ntok * G;
  const int p0 = kvl - q_len + first, p1 = p0 + ntok - 1;  // positions of this block's tokens
  const int nsplit = a.nsplit, split = blockIdx.y;
  if ((kvl <= 0 || p0 < 0) && nsplit > 1) {  // padding request: nothing seen, the merge writes zeros
    for (int row = tid; row < rows_valid; row += THREADS) {
      float* pp = a.parts + (((long long)(q_begin + first + row / G) * a.num_q + kh * G + row % G) * nsplit + split) * (dv + 2);
      pp[dv] = -INFINITY;
      pp[dv + 1] = 0.f;
    }
    return;
  }
  if (kvl <= 0 || p0 < 0) {                                // padding request: zeros
    for (int i = tid; i < rows_valid * dv; i += THREADS) {
      const int row = i / dv, d = i - row * dv;
      a.out[(long long)(q_begin + first + row / G) * a.out_stride + (long long)(kh * G + row % G) * dv + d] =
          __float2bfloat16_rn(0.f);
    }
    return;
  }
  const int key0 = W > 0 ? max(0, p0 - W + 1) : 0;
  const int nb = (W > 0 && a.pool > 0 && p1 - W + 1 > 0) ? (p1 - W + 1) / a.pool : 0;  // pooled entries in sight
  const int ptiles = (nb + WIN_N - 1) / WIN_N;
  const int tiles = ptiles + (p1 - key0 + WIN_N) / WIN_N;
  const int per_split = (tiles + nsplit - 1) / nsplit;
  const int t_begin = min(tiles, split * per_split), t_end = min(tiles, t_begin + per_split);
  const int* bt = a.block_table + (long long)a.req_slots[r] * a.max_pages;
  const int* pbt = nb > 0 ? a.p_block_table + (long long)a.req_slots[r] * a.p_max_pages : nullptr;
  const long long kv_row = (long long)num_kv * dk, v_row = (long long)num_kv * dv;
  const int kchunks = dk / 8, vchunks = dv / 8;

  for (int c = tid; c < WIN_M * kchunks; c += THREADS) {
    const int row = c / kchunks, ch = c - row * kchunks;
    const bool ok = row < rows_valid;
    const long long off =
        ok ? ((long long)(q_begin + first + row / G) * a.q_stride + (long long)(kh * G + row % G) * dk + ch * 8) : 0;
    win_cp_async_16(q_s + row * qs + ch * 16, a.q + off, ok);
  }
  win_commit();

  const int k_row0 = tid / kchunks, k_ch0 = tid % kchunks, k_drow = THREADS / kchunks, k_dch = THREADS % kchunks;
  const int v_row0 = tid / vchunks, v_ch0 = tid % vchunks, v_drow = THREADS / vchunks, v_dch = THREADS % vchunks;
  // Keys have two stages, value pages of their own ONE (with two, a block of 128-wide heads takes 87 KB and two
  // fit an SM; with one, three): tile t's values are asked for when tile t - 1's are used up, and awaited
  // between the softmax and P V of tile t.
  auto issue_values = [&](int tile) {
    const long long* slots = slot_s + (tile & 1) * WIN_N;
    const __nv_bfloat16* vc = (tile < ptiles ? a.pv : a.v_cache) + (long long)kh * dv;
    for (int row = v_row0, ch = v_ch0; row < WIN_N;) {
      const long long s = slots[row];
      const bool ok = s >= 0;
      win_cp_async_16(v_s + row * vs + ch * 16, vc + (ok ? s * v_row + ch * 8 : 0), ok);
      row += v_drow;
      ch += v_dch;
      if (ch >= vchunks) {
        ch -= vchunks;
        ++row;
      }
    }
  };
  auto issue = [&](int tile) {
    const int st = tile & 1;
    unsigned char* kbuf = k_s + st * WIN_N * qs;
    long long* slots = slot_s + st * WIN_N;
    const bool pooled = tile < ptiles;
    if (tid < WIN_N) {
      const int key = pooled ? tile * WIN_N + tid : key0 + (tile - ptiles) * WIN_N + tid;
      long long s = -1;
      if (pooled ? key < nb : key <= p1) {
        const int page = (pooled ? pbt : bt)[key / page_size];
        if (page < 0 || page >= (pooled ? a.p_num_pages : a.num_pages)) ullm_report(a.status, ULLM_STATUS_PAGE, r, page);
        else s = (long long)page * page_size + key % page_size;
      }
      slots[tid] = s;
    }
    __syncthreads();
    // a thread's 16-byte pieces are THREADS apart: (row, piece) steps by the quotient and remainder found once
    const __nv_bfloat16* kc = (pooled ? a.pk : a.k_cache) + (long long)kh * dk;
    for (int row = k_row0, ch = k_ch0; row < WIN_N;) {
      const long long s = slots[row];
      const bool ok = s >= 0;
      win_cp_async_16(kbuf + row * qs + ch * 16, kc + (ok ? s * kv_row + ch * 8 : 0), ok);
      row += k_drow;
      ch += k_dch;
      if (ch >= kchunks) {
        ch -= kchunks;
        ++row;
      }
    }
  };

  // a thread's two rows: wrow + lane / 4 and + 8
  const int wrow = rw * 16;
  const float log2e = 1.4426950408889634f;
  int pos[2], lo[2], nblk[2];
  float slope[2], slope_pos[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = wrow + (lane >> 2) + h * 8;
    const bool valid = row < rows_valid;
    pos[h] = valid ? p0 + row / G : -1;
    lo[h] = W > 0 ? pos[h] - W + 1 : 0;
    nblk[h] = (valid && a.pool > 0 && W > 0 && lo[h] > 0) ? lo[h] / a.pool : 0;
    slope[h] = (valid && a.slopes != nullptr) ? a.slopes[kh * G + row % G] * log2e : 0.f;
    slope_pos[h] = -slope[h] * (float)pos[h];
  }
  const bool has_slopes = a.slopes != nullptr;
  const bool warp_live = wrow < rows_valid;
  const int w_last = min(rows_valid, wrow + 16) - 1;
  const int wp_max = warp_live ? p0 + w_last / G : -1;
  const int wp_min = p0 + wrow / G;
  const int wp_lo = (warp_live && W > 0) ? wp_min - W + 1 : 0;
  const bool warp_full = wrow + 16 <= rows_valid;
  const int w_nblk = (warp_live && a.pool > 0 && W > 0 && wp_max - W + 1 > 0) ? (wp_max - W + 1) / a.pool : 0;
  const int c0 = cw * DVW;  // this warp's first value column

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[NT_O][4];
#pragma unroll
  for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

  // cp.async groups, oldest first: [Q] K(b) V(b) | K(b+1) | V(b+1) K(b+2) | ...  (the V groups only with value
  // pages of their own): at the top of tile t the two newest groups (V(t), K(t+1)) may be in flight, in front
  // of P V only K(t+1)
  if (t_begin < t_end) issue(t_begin);  // (its __syncthreads publishes the slots that issue_values reads)
  win_commit();
  if (v_own) {
    if (t_begin < t_end) issue_values(t_begin);
    win_commit();
  }
  for (int it = t_begin; it < t_end; ++it) {
    if (it + 1 < t_end) issue(it + 1);
    win_commit();
    if (v_own) win_wait<2>();
    else win_wait<1>();
    __syncthreads();
    const bool pooled = it < ptiles;
    const int kb = pooled ? it * WIN_N : key0 + (it - ptiles) * WIN_N;
    const bool live = warp_live && (pooled ? kb < w_nblk : (kb <= wp_max && kb + WIN_N - 1 >= wp_lo));
    const unsigned char* kbuf = k_s + (it & 1) * WIN_N * qs;
    const unsigned char* vbuf = v_own ? v_s : kbuf;
    float sc[NT_S][4];
    if (live) {
#pragma unroll
      for (int t = 0; t < NT_S; ++t) sc[t][0] = sc[t][1] = sc[t][2] = sc[t][3] = 0.f;
      const int mat = lane >> 3;
      const unsigned char* qp = q_s + (wrow + (mat & 1) * 8 + (lane & 7)) * qs + (mat >> 1) * 16;
      const unsigned char* kp = kbuf + ((mat >> 1) * 8 + (lane & 7)) * qs + (mat & 1) * 16;
      // with `ksplit` the column groups of a row group share the 16-wide steps of the key rows and add up their
      // partial scores through shared memory; otherwise each forms all of them
      const int ksteps = dk / 16;
      const int kk0 = (CW > 1 && a.ksplit) ? cw * ksteps / CW : 0;
      const int kk1 = (CW > 1 && a.ksplit) ? (cw + 1) * ksteps / CW : ksteps;
#pragma unroll(DKT > 0 ? (DKT / 16 <= 8 ? DKT / 16 : 4) : 2)
      for (int kk = kk0; kk < kk1; ++kk) {
        unsigned qa[4];
        win_ldsm4(qa[0], qa[1], qa[2], qa[3], qp + kk * 32);
#pragma unroll
        for (int t = 0; t < NT_S; t += 2) {
          unsigned b0, b1, b2, b3;
          win_ldsm4(b0, b1, b2, b3, kp + t * 8 * qs + kk * 32);
          win_mma(sc[t], qa, b0, b1);
          win_mma(sc[t + 1], qa, b2, b3);
        }
      }
      if (CW > 1 && a.ksplit) {
        float* mine = exch_s + ((rw * CW + cw) * 32) * 32 + lane;
#pragma unroll
        for (int t = 0; t < NT_S; ++t)
#pragma unroll
          for (int e = 0; e < 4; ++e) mine[(t * 4 + e) * 32] = sc[t][e];
        // (the row group's warps take this branch together: whether a tile is live depends on the rows only; the
        // buffer is written again after the tile's closing __syncthreads)
        asm volatile("bar.sync %0, %1;" ::"r"(rw + 1), "r"(CW * 32) : "memory");
#pragma unroll
        for (int o2 = 1; o2 < CW; ++o2) {
          const float* other = exch_s + ((rw * CW + (cw + o2) % CW) * 32) * 32 + lane;
#pragma unroll
          for (int t = 0; t < NT_S; ++t)
#pragma unroll
            for (int e = 0; e < 4; ++e) sc[t][e] += other[(t * 4 + e) * 32];
        }
      }
      // ---- scale, distance bias, mask: scores in units of log2 from here on ------------------
      const bool edge = pooled || !warp_full || kb + WIN_N - 1 > wp_min || (W > 0 && kb < wp_max - W + 1);
      if (has_slopes && !pooled) {
        // score * scale - slope (pos - key), as two multiply-adds per score
        const float kf = (float)(kb + (lane & 3) * 2);
#pragma unroll
        for (int t = 0; t < NT_S; ++t) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int h = e >> 1;
            sc[t][e] = fmaf(sc[t][e], a.scale_log2, fmaf(slope[h], kf + (float)(t * 8 + (e & 1)), slope_pos[h]));
          }
        }
        if (edge) {
#pragma unroll
          for (int t = 0; t < NT_S; ++t) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int key = kb + t * 8 + (lane & 3) * 2 + (e & 1), h = e >> 1;
              if (!(key <= pos[h] && key >= lo[h])) sc[t][e] = -INFINITY;
            }
          }
        }
      } else if (edge) {
#pragma unroll
        for (int t = 0; t < NT_S; ++t) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = kb + t * 8 + (lane & 3) * 2 + (e & 1), h = e >> 1;
            float s = sc[t][e] * a.scale_log2;
            bool seen;
            if (pooled) seen = key < nblk[h];
            else seen = key <= pos[h] && key >= lo[h];
            sc[t][e] = seen ? s : -INFINITY;
          }
        }
      } else {
#pragma unroll
        for (int t = 0; t < NT_S; ++t)
#pragma unroll
          for (int e = 0; e < 4; ++e) sc[t][e] *= a.scale_log2;
      }
      // ---- online softmax ---------------------------------------------------------------------
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int t = 0; t < NT_S; ++t) {
        mx[0] = fmaxf(mx[0], fmaxf(sc[t][0], sc[t][1]));
        mx[1] = fmaxf(mx[1], fmaxf(sc[t][2], sc[t][3]));
      }
      float alpha[2], neg_m[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        const float m_new = fmaxf(m[i], mx[i]);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;  // a row that has seen no key yet
        alpha[i] = win_ex2(m[i] - m_use);
        m[i] = m_new;
        l[i] *= alpha[i];
        neg_m[i] = -m_use;
      }
#pragma unroll
      for (int t = 0; t < NT_S; ++t) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p = win_ex2(sc[t][e] + neg_m[e >> 1]);
          sc[t][e] = p;
          l[e >> 1] += p;
        }
      }
      if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {  // (a maximum moved)
#pragma unroll
        for (int j = 0; j < NT_O; ++j) {
          o[j][0] *= alpha[0];
          o[j][1] *= alpha[0];
          o[j][2] *= alpha[1];
          o[j][3] *= alpha[1];
        }
      }
    }
    if (v_own) {
      win_wait<1>();
      __syncthreads();
    }
    if (live) {
      const int mat = lane >> 3;
      // ---- O += P V (this warp's columns) --------------------------------------------------------
      const unsigned char* vp = vbuf + ((mat & 1) * 8 + (lane & 7)) * vs + (c0 / 8 + (mat >> 1)) * 16;
#pragma unroll
      for (int ks = 0; ks < WIN_N / 16; ++ks) {
        unsigned pa[4];
        pa[0] = win_pack(sc[2 * ks][0], sc[2 * ks][1]);
        pa[1] = win_pack(sc[2 * ks][2], sc[2 * ks][3]);
        pa[2] = win_pack(sc[2 * ks + 1][0], sc[2 * ks + 1][1]);
        pa[3] = win_pack(sc[2 * ks + 1][2], sc[2 * ks + 1][3]);
#pragma unroll
        for (int j = 0; j < NT_O; j += 2) {
          if (c0 + j * 8 < dv) {
            unsigned b0, b1, b2, b3;
            win_ldsm4t(b0, b1, b2, b3, vp + ks * 16 * vs + j * 16);
            win_mma(o[j], pa, b0, b1);
            win_mma(o[j + 1], pa, b2, b3);
          }
        }
      }
    }
    __syncthreads();
    if (v_own) {
      if (it + 1 < t_end) issue_values(it + 1);
      win_commit();
    }
  }
  win_wait<0>();
  const int c = (lane & 3) * 2;
  const float out_scale = a.out_scale != 0.f ? a.out_scale : 1.f;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float ls = l[h];
    ls += __shfl_xor_sync(0xffffffffu, ls, 1);
    ls += __shfl_xor_sync(0xffffffffu, ls, 2);
    const float inv = (ls > 0.f ? 1.f / ls : 0.f) * out_scale;
    const int row = wrow + (lane >> 2) + h * 8;
    if (row < rows_valid && nsplit > 1) {
      float* pp = a.parts + (((long long)(q_begin + first + row / G) * a.num_q + kh * G + row % G) * nsplit + split) * (dv + 2);
#pragma unroll
      for (int j = 0; j < NT_O; ++j)
        if (c0 + j * 8 < dv) *reinterpret_cast<float2*>(pp + c0 + j * 8 + c) = make_float2(o[j][2 * h], o[j][2 * h + 1]);
      if (cw == 0 && (lane & 3) == 0) {
        pp[dv] = m[h];
        pp[dv + 1] = ls;
      }
    } else if (row < rows_valid) {
      const long long tok = q_begin + first + row / G;
      const long long col = (long long)(kh * G + row % G) * dv + c0 + c;
      __nv_bfloat16* op = a.out + tok * a.out_stride + col;
      const __nv_bfloat16* gp = a.gate != nullptr ? a.gate + tok * a.gate_stride + col : nullptr;
#pragma unroll
      for (int j = 0; j < NT_O; ++j) {
        if (c0 + j * 8 < dv) {
          float x = o[j][2 * h] * inv, y = o[j][2 * h + 1] * inv;
          if (gp != nullptr) {
            x /= 1.f + expf(-__bfloat162float(gp[j * 8]));
            y /= 1.f + expf(-__bfloat162float(gp[j * 8 + 1]));
          }
          *reinterpret_cast<unsigned*>(op + j * 8) = win_pack(x, y);
        }
      }
    }
  }
}

// One block per (token, head): the splits' accumulators, weighted by 2^(m_s - max m), over the weighted sums;
// then the scale, the gate and the one rounding.
__global__ void __launch_bounds__(128) window_merge_kernel(const WinArgs a) {
  __shared__ float w_s[64];
  __shared__ float inv_s;
  pdl_launch_dependents();
  pdl_wait();
  const long long th = blockIdx.x;
  const int dv = a.dv, nsplit = a.nsplit, tid = threadIdx.x;
  const float* pp = a.parts + th * nsplit * (dv + 2);
  if (tid < 32) {
    float mx = -INFINITY;
    for (int s = tid; s < nsplit; s += 32) mx = fmaxf(mx, pp[(long long)s * (dv + 2) + dv]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int s = tid; s < nsplit; s += 32) {
      const float ms = pp[(long long)s * (dv + 2) + dv];
      const float w = ms == -INFINITY ? 0.f : win_ex2(ms - mx);
      w_s[s] = w;
      sum += w * pp[(long long)s * (dv + 2) + dv + 1];
    }
    sum = warp_sum(sum);
    if (tid == 0) inv_s = (sum > 0.f ? 1.f / sum : 0.f) * (a.out_scale != 0.f ? a.out_scale : 1.f);
  }
  __syncthreads();
  const long long tok = th / a.num_q;
  const int head = (int)(th - tok * a.num_q);
  __nv_bfloat16* op = a.out + tok * a.out_stride + (long long)head * dv;
  const __nv_bfloat16* gp = a.gate != nullptr ? a.gate + tok * a.gate_stride + (long long)head * dv : nullptr;
  for (int e = tid; e < dv; e += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < nsplit; ++s)
      if (w_s[s] > 0.f) acc += w_s[s] * pp[(long long)s * (dv + 2) + e];
    acc *= inv_s;
    if (gp != nullptr) acc /= 1.f + expf(-__bfloat162float(gp[e]));
    op[e] = __float2bfloat16_rn(acc);
  }
}

#define WIN_SMEM_LIMIT (227 * 1024)
#define WIN_MAX_SPLITS 64

template <int DVW, int CW, int RW, int DKT = 0>
static int launch_window(WinArgs a, int tokens, long long smem, cudaStream_t st) {
  if (CW > 1 && smem + win_exchange_bytes(a.dv) <= WIN_SMEM_LIMIT) {
    a.ksplit = 1;
    smem += win_exchange_bytes(a.dv);
  }
  static long long attr_bytes = 0;  // (one per instantiation) the largest size the attribute was set for
  if (smem > attr_bytes) {
    if (cudaFuncSetAttribute(window_attention_kernel<DVW, CW, RW, DKT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return ULLM_ERR_LAUNCH;
    cudaFuncSetAttribute(window_attention_kernel<DVW, CW, RW, DKT>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    attr_bytes = smem;
  }
  const int tpt = RW * 16 / (a.num_q / a.num_kv);
  // at most ceil(tokens / tpt) + num_requests token tiles exist, however the tokens are spread
  const long long blocks = ((long long)(tokens + tpt - 1) / tpt + a.num_requests) * a.num_kv;
  if (blocks > 0x7fffffffLL) return ULLM_ERR_BAD_SIZE;
  const int rc = ullm_launch_kernel(window_attention_kernel<DVW, CW, RW, DKT>, dim3((unsigned)blocks, (unsigned)a.nsplit),
                                    dim3(RW * CW * 32), (size_t)smem, st, a);
  if (rc != ULLM_OK || a.nsplit <= 1) return rc;
  return ullm_launch_kernel(window_merge_kernel, dim3((unsigned)((long long)tokens * a.num_q)), dim3(128), 0, st, a);
}

// Sizes this kernel takes (bfloat16): key rows and values multiples of 16, values up to 512, at most 64 query
// heads per kv head, and tiles that fit the shared memory (key rows up to 576 with values inside them).
extern "C" int ullm_window_attention_supported(int dk, int dv, int num_q, int num_kv, int values_in_keys) {
  if (dk <= 0 || dv <= 0 || num_q <= 0 || num_kv <= 0 || num_q % num_kv) return 0;
  if (dk % 16 || dv % 16 || dv > 512 || num_q / num_kv > WIN_MAX_GROUP) return 0;
  if (values_in_keys && dv > dk) return 0;
  return win_smem_bytes(dk, dv, !values_in_keys) <= WIN_SMEM_LIMIT;
}

// `v_cache` null: values inside the key rows (and then `pv` null too).  `slopes` (32-bit [num_q]) or null;
// `pool` > 0 with the pooled pages `pk` (`pv`) and their block table; `gate` or null; `out_scale` 0 = 1.
// `nsplit` > 1 (at most 64) with `parts` (32-bit, tokens x num_q x nsplit x (dv + 2)): a block's key tiles are
// cut into nsplit runs that run side by side and are merged by a second launch (steps of few rows).
// q rows, page rows, `out` and `gate` rows must start on 16- (q, pages) and 4-byte (out) boundaries.
extern "C" int ullm_window_attention(const void* q, long long q_row_stride, void* out, long long out_stride,
                                     const void* k_cache, const void* v_cache, const int* block_table, int max_pages,
                                     const int* req_slots, const int* cu_q, const int* kv_len, int tokens,
                                     int num_requests, int num_q, int num_kv, int dk, int dv, int page_size, int window,
                                     float scale, long long num_pages, int* status, void* stream, const float* slopes,
                                     int pool, const void* pk, const void* pv, const int* p_block_table,
                                     int p_max_pages, long long p_num_pages, const void* gate, long long gate_stride,
                                     float out_scale, int nsplit, float* parts) {
  cudaStream_t st = (cudaStream_t)stream;
  if (tokens < 0 || num_requests <= 0 || page_size <= 0 || max_pages <= 0 || window < 0 || pool < 0)
    return ULLM_ERR_BAD_SIZE;
  if (!ullm_window_attention_supported(dk, dv, num_q, num_kv, v_cache == nullptr)) return ULLM_ERR_UNSUPPORTED;
  if (pool > 0 && (window <= 0 || pk == nullptr || p_block_table == nullptr || p_max_pages <= 0 || slopes != nullptr ||
                   (pv == nullptr) != (v_cache == nullptr)))
    return ULLM_ERR_UNSUPPORTED;
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)pk | (uintptr_t)pv) & 15) return ULLM_ERR_BAD_SIZE;
  if (q_row_stride % 8 || ((uintptr_t)out & 3) || out_stride % 2 || out_stride < (long long)num_q * dv)
    return ULLM_ERR_BAD_SIZE;
  if (nsplit < 1 || nsplit > WIN_MAX_SPLITS || (nsplit > 1 && parts == nullptr) || ((uintptr_t)parts & 7))
    return ULLM_ERR_BAD_SIZE;
  if ((long long)tokens * num_q > 0x7fffffffLL) return ULLM_ERR_BAD_SIZE;
  if (tokens == 0) return ULLM_OK;
  WinArgs a = {};
  a.q = (const __nv_bfloat16*)q;
  a.q_stride = q_row_stride;
  a.out = (__nv_bfloat16*)out;
  a.out_stride = out_stride;
  a.k_cache = (const __nv_bfloat16*)k_cache;
  a.v_cache = (const __nv_bfloat16*)v_cache;
  a.block_table = block_table;
  a.max_pages = max_pages;
  a.num_pages = num_pages;
  a.req_slots = req_slots;
  a.cu_q = cu_q;
  a.kv_len = kv_len;
  a.num_requests = num_requests;
  a.num_q = num_q;
  a.num_kv = num_kv;
  a.dk = dk;
  a.dv = dv;
  a.page_size = page_size;
  a.window = window;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.slopes = slopes;
  a.pool = pool;
  a.pk = (const __nv_bfloat16*)pk;
  a.pv = (const __nv_bfloat16*)pv;
  a.p_block_table = p_block_table;
  a.p_max_pages = p_max_pages;
  a.p_num_pages = p_num_pages;
  a.gate = (const __nv_bfloat16*)gate;
  a.gate_stride = gate_stride;
  a.out_scale = out_scale;
  a.status = status;
  a.nsplit = nsplit;
  a.parts = parts;
  const long long smem = win_smem_bytes(dk, dv, v_cache != nullptr);
  // the sizes of the usual head shapes (64, 128; latents of 384 + 64 and 512 + 64) as constants
  if (dk == 64 && dv == 64) return launch_window<64, 1, 4, 64>(a, tokens, smem, st);
  if (dk == 128 && dv == 128) return launch_window<128, 1, 4, 128>(a, tokens, smem, st);
  if (dk == 448 && dv == 384) return launch_window<128, 3, 4, 448>(a, tokens, smem, st);
  if (dk == 576 && dv == 512) return launch_window<256, 2, 4, 576>(a, tokens, smem, st);
  if (dv <= 64) return launch_window<64, 1, 4>(a, tokens, smem, st);
  if (dv <= 128) return launch_window<128, 1, 4>(a, tokens, smem, st);
  if (dv <= 256) return launch_window<128, 2, 4>(a, tokens, smem, st);
  if (dv <= 384) return launch_window<128, 3, 4>(a, tokens, smem, st);
  return launch_window<256, 2, 4>(a, tokens, smem, st);
}
