// Grouped-query attention over a paged cache with a choice of mask and of weight rule, keys and
// values of different widths, any sizes, any cut; and the kernel that prepares its step.
//
//   mask (besides j <= p):  0 causal;  1 window: p - j < size;  2 chunk: floor(j/size) == floor(p/size)
//   weights:  0 softmax;  1 softmax with one more member of score 0 that has no value,
//             w_j = exp(s_j) / (1 + sum exp(s_j));  2 sigmoid(s_j + bias[head]), nothing normalised
//   s_j = (q . k_j) * scale,  kv_head = q_head / (n_q / n_kv),  out = sum_j w_j v_j
//
// A token's row of the fused projection is [q heads x dk | k heads x dk | v heads x dv].
//
// leone_attention_prepare: per token, in fp32: an optional RMS norm of q and of k (per head with
// one weight [dk] for all heads, or over all of a token's query heads at once and over all its key
// heads at once with weights [n_q dk] and [n_kv dk]; the weight multiplies directly), then the
// rotation of the first rot_dims elements of every q and k head by position * freq[pair] (pair i is
// elements (i, i + rot_dims/2), or (2i, 2i + 1) with `adjacent`; angle, cos and sin formed in fp32),
// q and k written back in place, k into the key page and v into the value page of the token.
//
// leone_attention_masked: one block per (token, query head); scores and weights in fp32, online
// over tiles of 128 keys in ascending order.  The softmax with the silent member is the ordinary
// online softmax started from (maximum 0, denominator 1, sum 0).  A row's arithmetic depends on its
// own sequence only, so results do not depend on how tokens were cut into steps or batched.
#include "common.cuh"

namespace leone {

constexpr int kPrepThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kPrepThreads)
attention_prepare_kernel(T* __restrict__ qkv, int row_stride, int n_q, int n_kv, int dk, int dv, int norm_mode,
                         const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                         const float* __restrict__ freqs, int rot_dims, int adjacent,
                         const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                         const int* __restrict__ block_table, int table_width, int n_seqs,
                         T* __restrict__ k_pool, T* __restrict__ v_pool, int num_pages, int page_tokens,
                         int* status) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  const int heads = n_q + n_kv;                  // the heads that are normed and rotated
  float* buf = smem;                             // [heads * dk] q then k, fp32
  float* head_ss = buf + (size_t)heads * dk;     // [heads] sums of squares, then the factors
  float* cs = head_ss + heads;                   // [rot_dims] cos, sin per pair
  const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, warps = kPrepThreads / 32;
  T* row = qkv + (size_t)t * row_stride;
  const int pos = positions[t];
  const int qk = heads * dk;
  if (pos < 0) {
    if (tid == 0) set_status(status, kBadPosition, t, pos);
    return;
  }
  for (int c = tid; c < qk; c += kPrepThreads) buf[c] = to_float<T>(row[c]);
  const int half = rot_dims >> 1;
  for (int i = tid; i < half; i += kPrepThreads) {
    const float angle = (float)pos * freqs[i];
    float s, c;
    sincosf(angle, &s, &c);
    cs[2 * i] = c;
    cs[2 * i + 1] = s;
  }
  __syncthreads();
  if (norm_mode != 0) {
    for (int h = warp; h < heads; h += warps) {
      float ss = 0.f;
      for (int c = lane; c < dk; c += 32) ss = fmaf(buf[h * dk + c], buf[h * dk + c], ss);
      ss = warp_sum(ss);
      if (lane == 0) head_ss[h] = ss;
    }
    __syncthreads();
    if (tid == 0) {
      if (norm_mode == 2) {            // all query heads together, all key heads together
        float sq = 0.f, sk = 0.f;
        for (int h = 0; h < n_q; ++h) sq += head_ss[h];
        for (int h = n_q; h < heads; ++h) sk += head_ss[h];
        const float rq = 1.f / sqrtf(sq / (float)(n_q * dk) + eps), rk = 1.f / sqrtf(sk / (float)(n_kv * dk) + eps);
        for (int h = 0; h < heads; ++h) head_ss[h] = h < n_q ? rq : rk;
      } else {
        for (int h = 0; h < heads; ++h) head_ss[h] = 1.f / sqrtf(head_ss[h] / (float)dk + eps);
      }
    }
    __syncthreads();
    for (int c = tid; c < qk; c += kPrepThreads) {
      const int h = c / dk, e = c - h * dk;
      const float* w = h < n_q ? q_w : k_w;
      const int wi = norm_mode == 2 ? (h < n_q ? c : c - n_q * dk) : e;
      buf[c] = buf[c] * head_ss[h] * w[wi];
    }
    __syncthreads();
  }
  // where the token's key and value rows go
  long long key_at = -1, value_at = -1;
  if (k_pool != nullptr) {
    const int s = seq_of_token[t];
    if (s < 0 || s >= n_seqs) {
      if (tid == 0) set_status(status, kBadSequence, t, s);
      return;
    }
    const int blk = pos / page_tokens;
    const int page = blk < table_width ? block_table[(size_t)s * table_width + blk] : -1;
    if (page < 0 || page >= num_pages) {
      if (tid == 0) set_status(status, kBadPage, t, page, pos);
      return;
    }
    const long long slot = (long long)page * n_kv * page_tokens + (pos % page_tokens);
    key_at = slot * dk;          // kv head h adds h * page_tokens * dk
    value_at = slot * dv;
  }
  for (int c = tid; c < qk; c += kPrepThreads) {
    const int h = c / dk, e = c - h * dk;
    float v = buf[c];
    if (e < rot_dims) {
      const int pair = adjacent ? e >> 1 : (e < half ? e : e - half);
      const bool first = adjacent ? (e & 1) == 0 : e < half;
      const float a = buf[h * dk + (adjacent ? 2 * pair : pair)], b = buf[h * dk + (adjacent ? 2 * pair + 1 : pair + half)];
      const float co = cs[2 * pair], si = cs[2 * pair + 1];
      v = first ? a * co - b * si : b * co + a * si;
    }
    const T o = from_float<T>(v);
    row[c] = o;
    if (h >= n_q && key_at >= 0) k_pool[key_at + (long long)(h - n_q) * page_tokens * dk + e] = o;
  }
  if (value_at >= 0) {
    const T* vrow = row + qk;
    for (int c = tid; c < n_kv * dv; c += kPrepThreads) {
      const int h = c / dv, e = c - h * dv;
      v_pool[value_at + (long long)h * page_tokens * dv + e] = vrow[c];
    }
  }
}

constexpr int kMaskedThreads = 128;
constexpr int kMaskedAcc = 8;          // value width <= 1024

// First key a query at `pos` sees.
__device__ __forceinline__ int first_seen(int mask, int size, int pos) {
  if (mask == 1) return max(0, pos - size + 1);
  if (mask == 2) return (pos / size) * size;
  return 0;
}

template <typename T>
__global__ void __launch_bounds__(kMaskedThreads)
attention_masked_kernel(const T* __restrict__ qkv, int row_stride, T* __restrict__ out, int out_stride,
                        const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                        const int* __restrict__ block_table, int table_width,
                        const int* __restrict__ seq_of_token, const int* __restrict__ positions, int n_q, int n_kv,
                        int dk, int dv, float scale, int mask, int mask_size, int weights,
                        const float* __restrict__ bias, int page_tokens, int num_pages, int n_seqs, int* status) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  long long* off_s = (long long*)smem;                // [128] slot of the key among its pool's rows
  float* p_s = smem + 2 * kMaskedThreads;             // [128]
  float* q_s = p_s + kMaskedThreads;                  // [dk]
  __shared__ float scratch[33];
  __shared__ int bad;

  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int pos = positions[t], s = seq_of_token[t];
  const int kvh = h / (n_q / n_kv);
  T* dst = out + (size_t)t * out_stride + (size_t)h * dv;
  if (tid == 0) bad = 0;
  if (s < 0 || s >= n_seqs || pos < 0) {
    if (tid == 0) set_status(status, s < 0 || s >= n_seqs ? kBadSequence : kBadPosition, t, s < 0 || s >= n_seqs ? s : pos);
    for (int c = tid; c < dv; c += kMaskedThreads) dst[c] = from_float<T>(0.f);
    return;
  }
  const T* q = qkv + (size_t)t * row_stride + (size_t)h * dk;
  for (int c = tid; c < dk; c += kMaskedThreads) q_s[c] = to_float<T>(q[c]);
  __syncthreads();

  const int lo = first_seen(mask, mask_size, pos);
  const float b = (weights == 2 && bias != nullptr) ? bias[h] : 0.f;
  // the silent member of score 0: the running maximum starts at 0 and the denominator at exp(0 - 0)
  float m_run = weights == 1 ? 0.f : -INFINITY, l_run = weights == 1 ? 1.f : 0.f;
  float acc[kMaskedAcc];
#pragma unroll
  for (int i = 0; i < kMaskedAcc; ++i) acc[i] = 0.f;

  for (int j0 = lo; j0 <= pos; j0 += kMaskedThreads) {
    const int j = j0 + tid;
    float score = -INFINITY;
    long long slot = -1;
    if (j <= pos) {
      const int blk = j / page_tokens;
      const int page = blk < table_width ? block_table[(size_t)s * table_width + blk] : -1;
      if (page < 0 || page >= num_pages) {
        set_status(status, kBadPage, t, page, j);
        bad = 1;
      } else {
        slot = ((long long)page * n_kv + kvh) * page_tokens + (j % page_tokens);
        const T* krow = k_pool + slot * dk;
        float dot = 0.f;
        for (int c = 0; c < dk; ++c) dot = fmaf(q_s[c], to_float<T>(krow[c]), dot);
        score = dot * scale;
      }
    }
    off_s[tid] = slot;
    float alpha = 1.f;
    if (weights == 2) {
      p_s[tid] = slot >= 0 ? 1.f / (1.f + expf(-(score + b))) : 0.f;
      __syncthreads();
    } else {
      const float tile_max = block_max(score, scratch);
      const float m_new = fmaxf(m_run, tile_max);
      const float p = slot >= 0 ? expf(score - m_new) : 0.f;
      p_s[tid] = p;
      const float tile_sum = block_sum(p, scratch);   // also orders p_s/off_s writes before reads
      alpha = m_run == -INFINITY ? 0.f : expf(m_run - m_new);
      l_run = l_run * alpha + tile_sum;
      m_run = m_new;
    }
    const int count = min(kMaskedThreads, pos - j0 + 1);
#pragma unroll
    for (int i = 0; i < kMaskedAcc; ++i) {
      const int c = tid + i * kMaskedThreads;
      if (c < dv) {
        float a = acc[i] * alpha;
        for (int jj = 0; jj < count; ++jj) {
          const long long r = off_s[jj];
          if (r >= 0) a = fmaf(p_s[jj], to_float<T>(v_pool[r * dv + c]), a);
        }
        acc[i] = a;
      }
    }
    __syncthreads();
  }
  float inv = weights == 2 ? 1.f : (l_run > 0.f ? 1.f / l_run : 0.f);
  if (bad) inv = 0.f;
#pragma unroll
  for (int i = 0; i < kMaskedAcc; ++i) {
    const int c = tid + i * kMaskedThreads;
    if (c < dv) dst[c] = from_float<T>(acc[i] * inv);
  }
}

}  // namespace leone

using namespace leone;

// norm_mode: 0 none, 1 per head (weights [dk]), 2 over all query heads / all key heads (weights
// [n_q dk], [n_kv dk]); weights fp32.  freqs: fp32 [rot_dims / 2] or null (no rotation).
// k_pool null: nothing is written into pages (a layer that reads another layer's cache).
extern "C" int leone_attention_prepare(int dtype, void* qkv, int row_stride, int n_tokens, int n_q, int n_kv, int dk,
                                       int dv, int norm_mode, const float* q_w, const float* k_w, float eps,
                                       const float* freqs, int rot_dims, int adjacent, const int* positions,
                                       const int* seq_of_token, const int* block_table, int table_width, int n_seqs,
                                       void* k_pool, void* v_pool, int num_pages, int page_tokens, int* status,
                                       cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (dk <= 0 || dv <= 0 || n_q <= 0 || n_kv <= 0 || norm_mode < 0 || norm_mode > 2) return kRefusedSize;
  if (norm_mode != 0 && (q_w == nullptr || k_w == nullptr)) return kRefusedSize;
  if (freqs == nullptr) rot_dims = 0;
  if (rot_dims < 0 || rot_dims > dk || (rot_dims & 1)) return kRefusedSize;
  if (k_pool != nullptr && (v_pool == nullptr || page_tokens <= 0 || table_width <= 0)) return kRefusedSize;
  if (row_stride < (n_q + n_kv) * dk + n_kv * dv) return kRefusedSize;
  const size_t smem = ((size_t)(n_q + n_kv) * dk + (n_q + n_kv) + rot_dims + 2) * sizeof(float);
  if (smem > 200 * 1024) return kRefusedSize;
#define LAUNCH(T)                                                                                              \
  {                                                                                                            \
    if (smem > 48 * 1024)                                                                                      \
      cudaFuncSetAttribute(attention_prepare_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    return launch_kernel(attention_prepare_kernel<T>, dim3(n_tokens), dim3(kPrepThreads), smem, stream, (T*)qkv, \
                         row_stride, n_q, n_kv, dk, dv, norm_mode, q_w, k_w, eps, freqs, rot_dims, adjacent,      \
                         positions, seq_of_token, block_table, table_width, n_seqs, (T*)k_pool, (T*)v_pool,      \
                         num_pages, page_tokens, status);                                                        \
  }
  if (dtype == 0) LAUNCH(float);
  if (dtype == 1) LAUNCH(__nv_bfloat16);
#undef LAUNCH
  return kRefusedDtype;
}

extern "C" int leone_attention_masked(int dtype, const void* qkv, int row_stride, void* out, int out_stride,
                                      const void* k_pool, const void* v_pool, const int* block_table,
                                      int table_width, const int* seq_of_token, const int* positions, int n_tokens,
                                      int n_q, int n_kv, int dk, int dv, float scale, int mask, int mask_size,
                                      int weights, const float* bias, int page_tokens, int num_pages, int n_seqs,
                                      int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (dk <= 0 || dk > 8192 || dv <= 0 || dv > kMaskedThreads * kMaskedAcc || n_q <= 0 || n_kv <= 0 ||
      n_q % n_kv != 0 || n_q > 65535 || page_tokens <= 0 || table_width <= 0)
    return kRefusedSize;
  if (mask < 0 || mask > 2 || weights < 0 || weights > 2 || (mask != 0 && mask_size <= 0)) return kRefusedSize;
  dim3 grid(n_tokens, n_q);
  const size_t smem = (size_t)(dk + kMaskedThreads) * sizeof(float) + kMaskedThreads * sizeof(long long) + 8;
#define LAUNCH(T)                                                                                               \
  return launch_kernel(attention_masked_kernel<T>, grid, dim3(kMaskedThreads), smem, stream, (const T*)qkv,      \
                       row_stride, (T*)out, out_stride, (const T*)k_pool, (const T*)v_pool, block_table,         \
                       table_width, seq_of_token, positions, n_q, n_kv, dk, dv, scale, mask, mask_size, weights, \
                       bias, page_tokens, num_pages, n_seqs, status)
  if (dtype == 0) LAUNCH(float);
  if (dtype == 1) LAUNCH(__nv_bfloat16);
#undef LAUNCH
  return kRefusedDtype;
}
