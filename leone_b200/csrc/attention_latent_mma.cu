// Attention through a cached latent on tensor cores (bfloat16), for prompt portions and decode.
//
// All query heads of a token share the cache rows [c | r] as keys and c as values, so the heads of
// one token are the 16 rows of an MMA tile: a group of four warps owns one token (and up to 16 of
// its heads; a block has one such group, or four for prompt portions, whose consecutive tokens share
// most of their keys) and walks the token's keys in tiles of 64 rows, which it copies once from the pages
// into shared memory and uses twice: as K (all dk elements) for S = Q K^T and as V (the first dv
// elements) for O += P V.  Warp w computes the scores of keys 16w..16w+15 of the tile; the rows'
// maxima and sums cross the warps through shared memory (fp32 online softmax, the per-head sink as
// the first score); P goes to shared memory as bfloat16 and every warp multiplies it with its
// quarter of the value columns.  O stays in registers (16 x dv/4 fp32 per warp).  A step of few tokens
// (decode) splits each token's keys over several blocks, which leave (O, m, l) in scratch for a merge
// kernel that also adds the sink and applies the gate.
//
// Sizes: dk a multiple of 16, dv = 32 * NT with NT in {2, 4, 6, 8, 12, 16}; other sizes take the
// any-size kernel of attention_latent.cu.
#include "common.cuh"

namespace leone {

constexpr int kTile = 64;         // keys per tile
constexpr int kMmaThreads = 128;

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n cp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// G tokens per block (G warp groups of four warps): consecutive tokens of a sequence share most of
// their keys, so one copy of a key tile serves all G.  Tokens of the block that belong to different
// sequences are served in passes, one run of same-sequence tokens at a time.
template <typename TS, int NT, int G>
__global__ void __launch_bounds__(kMmaThreads * G)
attention_latent_mma_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                            const __nv_bfloat16* __restrict__ pool, const int* __restrict__ block_table,
                            int table_width, const int* __restrict__ seq_of_token,
                            const int* __restrict__ positions, int n_tokens, int heads, int dk, float scale,
                            int window, const TS* __restrict__ sink, const __nv_bfloat16* __restrict__ gate, int ldg,
                            int page_tokens, int num_pages, int n_seqs, int splits, float* __restrict__ partial,
                            int* status) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  constexpr int dv = 32 * NT;
  constexpr int kThreads = kMmaThreads * G;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int pitch = dk * 2 + 16;                       // bytes per row of K and Q: no two of 8 rows share a bank
  constexpr int p_pitch = kTile * 2 + 16;
  const int group_bytes = 16 * pitch + 16 * p_pitch + 128 * (int)sizeof(float);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wg = warp >> 2, w4 = warp & 3, gtid = tid & (kMmaThreads - 1);
  unsigned char* k_s = smem_raw;                       // [kTile][pitch], shared by the groups
  unsigned char* q_s = k_s + kTile * pitch + wg * group_bytes;     // [16][pitch]
  unsigned char* p_s = q_s + 16 * pitch;               // [16][p_pitch]
  float* red_max = reinterpret_cast<float*>(p_s + 16 * p_pitch);   // [4][16]
  float* red_sum = red_max + 64;                                   // [4][16]
  __shared__ int bad;
  __shared__ int tok_seq[G], tok_pos[G];
  const int h0 = blockIdx.y * 16;
  const int g = lane >> 2, tq = lane & 3;
  const int t = blockIdx.x * G + wg;
  const int nh = min(16, heads - h0);
  if (tid == 0) bad = 0;
  if (tid < G) {
    const int tt = blockIdx.x * G + tid;
    int sq = -1, ps = -1;
    if (tt < n_tokens) {
      sq = seq_of_token[tt];
      ps = positions[tt];
      if (sq < 0 || sq >= n_seqs || ps < 0) {
        set_status(status, sq < 0 || sq >= n_seqs ? kBadSequence : kBadPosition, tt, ps);
        sq = -1;
      }
    }
    tok_seq[tid] = sq;
    tok_pos[tid] = ps;
  }
  __syncthreads();
  const int pos = tok_pos[wg], s_mine = tok_seq[wg];
  // with several splits (G == 1), this block's rows of the partial results: [16][dv + 2] floats (O, m, l)
  float* mine = splits > 1 ? partial + (((size_t)t * gridDim.y + blockIdx.y) * splits + blockIdx.z) * 16 * (dv + 2)
                           : nullptr;
  const uint32_t k_base = (uint32_t)__cvta_generic_to_shared(k_s);
  const uint32_t q_base = (uint32_t)__cvta_generic_to_shared(q_s);
  const uint32_t p_base = (uint32_t)__cvta_generic_to_shared(p_s);
  const int chunks = dk / 8;                           // 16-byte pieces per row
  // the token's query rows (heads past the last, and a token that is not there, are zero rows)
  for (int i = gtid; i < 16 * chunks; i += kMmaThreads) {
    const int r = i / chunks, c = i - r * chunks;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < nh && s_mine >= 0) v = *reinterpret_cast<const uint4*>(q + ((size_t)t * heads + h0 + r) * dk + c * 8);
    *reinterpret_cast<uint4*>(q_s + r * pitch + c * 16) = v;
  }
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  // running maximum and denominator of the thread's two rows (g and g + 8); the sink is a score
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  if (sink != nullptr && splits == 1) {            // with several splits the merge adds the sink
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = g + 8 * i;
      if (r < nh) {
        m_run[i] = to_float<TS>(sink[h0 + r]);
        l_run[i] = 1.f;
      }
    }
  }
  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[n][i] = 0.f;

  for (int p0 = 0; p0 < G;) {
    // the run of tokens p0..e-1 of one sequence, and the keys any of them reads
    const int sq = tok_seq[p0];
    int e = p0 + 1;
    while (e < G && sq >= 0 && tok_seq[e] == sq) ++e;
    if (sq < 0) {
      p0 = e;
      continue;
    }
    const bool active = wg >= p0 && wg < e;
    int run_lo = 0x7fffffff, run_hi = -1;
    for (int i = p0; i < e; ++i) {
      const int pi = tok_pos[i];
      run_lo = min(run_lo, window > 0 ? max(0, pi - window + 1) : 0);
      run_hi = max(run_hi, pi);
    }
    int j_first = run_lo, j_last = run_hi;
    if (splits > 1) {
      const int tiles = (run_hi - run_lo) / kTile + 1;
      const int per = (tiles + splits - 1) / splits;
      j_first = run_lo + (int)blockIdx.z * per * kTile;
      j_last = min(run_hi, j_first + per * kTile - 1);
    }
    for (int j0 = j_first; j0 <= j_last; j0 += kTile) {
      __syncthreads();                                 // the tile before is no longer read
      // copy the tile's rows from their pages (rows past the run's last position are zero)
      for (int r = warp; r < kTile; r += 4 * G) {
        const int j = j0 + r;
        const __nv_bfloat16* src = nullptr;
        if (j <= run_hi) {
          const int blk = j / page_tokens;
          const int page = blk < table_width ? block_table[(size_t)sq * table_width + blk] : -1;
          if (page < 0 || page >= num_pages) {
            if (lane == 0) {
              set_status(status, kBadPage, blockIdx.x * G + p0, page, j);
              bad = 1;
            }
          } else {
            src = pool + ((size_t)page * page_tokens + (j % page_tokens)) * dk;
          }
        }
        unsigned char* dst = k_s + r * pitch;
        if (src != nullptr) {
          for (int c = lane; c < chunks; c += 32) cp_async16(k_base + r * pitch + c * 16, src + c * 8);
        } else {
          for (int c = lane; c < chunks; c += 32) *reinterpret_cast<uint4*>(dst + c * 16) = make_uint4(0, 0, 0, 0);
        }
      }
      cp_async_wait_all();
      __syncthreads();
      // S for this warp's 16 keys: two tiles of 8 keys
      float sc[2][4];
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) sc[n][i] = 0.f;
      if (active) {
        const uint32_t a_addr = q_base + (lane & 15) * pitch + (lane >> 4) * 16;
        const int mi = lane >> 3;
        const uint32_t b_addr = k_base + (w4 * 16 + (lane & 7) + (mi >> 1) * 8) * pitch + (mi & 1) * 16;
        for (int kk = 0; kk < dk / 16; ++kk) {
          uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
          ldsm_x4(a_addr + kk * 32, a0, a1, a2, a3);
          ldsm_x4(b_addr + kk * 32, b0, b1, b2, b3);
          mma_bf16(sc[0], a0, a1, a2, a3, b0, b1);
          mma_bf16(sc[1], a0, a1, a2, a3, b2, b3);
        }
      }
      // scale, mask (the token's own keys lo..pos), the rows' maxima over this warp's keys
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int key = j0 + w4 * 16 + n * 8 + 2 * tq + (i & 1);
          const float v = (active && key <= pos && key >= lo) ? sc[n][i] * scale : -INFINITY;
          sc[n][i] = v;
          mx[i >> 1] = fmaxf(mx[i >> 1], v);
        }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
      }
      if (tq == 0) {
        red_max[w4 * 16 + g] = mx[0];
        red_max[w4 * 16 + g + 8] = mx[1];
      }
      __syncthreads();
      float m_new[2], alpha[2], sum[2] = {0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = g + 8 * i;
        const float tile_max = fmaxf(fmaxf(red_max[r], red_max[16 + r]), fmaxf(red_max[32 + r], red_max[48 + r]));
        m_new[i] = fmaxf(m_run[i], tile_max);
        alpha[i] = m_run[i] == -INFINITY ? 0.f : expf(m_run[i] - m_new[i]);
      }
      // P = exp(S - m) as bfloat16 into shared memory; the denominator is summed in fp32 before rounding
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        float p[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          p[i] = sc[n][i] == -INFINITY ? 0.f : expf(sc[n][i] - m_new[i >> 1]);
          sum[i >> 1] += p[i];
        }
        const int col = w4 * 16 + n * 8 + 2 * tq;
        *reinterpret_cast<uint32_t*>(p_s + g * p_pitch + col * 2) = pack_bf16(p[0], p[1]);
        *reinterpret_cast<uint32_t*>(p_s + (g + 8) * p_pitch + col * 2) = pack_bf16(p[2], p[3]);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
        sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
      }
      if (tq == 0) {
        red_sum[w4 * 16 + g] = sum[0];
        red_sum[w4 * 16 + g + 8] = sum[1];
      }
      __syncthreads();
      if (active) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int r = g + 8 * i;
          l_run[i] = l_run[i] * alpha[i] + ((red_sum[r] + red_sum[16 + r]) + (red_sum[32 + r] + red_sum[48 + r]));
          m_run[i] = m_new[i];
        }
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          o[n][0] *= alpha[0];
          o[n][1] *= alpha[0];
          o[n][2] *= alpha[1];
          o[n][3] *= alpha[1];
        }
        // O += P V for this warp's quarter of the value columns
        const uint32_t a_addr = p_base + (lane & 15) * p_pitch + (lane >> 4) * 16;
        const int mi = lane >> 3;
        const uint32_t v_addr = k_base + ((lane & 7) + (mi & 1) * 8) * pitch + (w4 * (dv / 4) + (mi >> 1) * 8) * 2;
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk) {
          uint32_t a0, a1, a2, a3;
          ldsm_x4(a_addr + kk * 32, a0, a1, a2, a3);
#pragma unroll
          for (int n = 0; n < NT; n += 2) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4_trans(v_addr + kk * 16 * pitch + n * 16, b0, b1, b2, b3);
            mma_bf16(o[n], a0, a1, a2, a3, b0, b1);
            mma_bf16(o[n + 1], a0, a1, a2, a3, b2, b3);
          }
        }
      }
    }
    p0 = e;
  }
  __syncthreads();
  const int failed = bad;
  if (t >= n_tokens) return;
  if (mine != nullptr) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float* row = mine + (g + 8 * i) * (dv + 2);
#pragma unroll
      for (int n = 0; n < NT; ++n)
        *reinterpret_cast<float2*>(row + w4 * (dv / 4) + n * 8 + 2 * tq) = make_float2(o[n][2 * i], o[n][2 * i + 1]);
      if (w4 == 0 && tq == 0) {
        row[dv] = s_mine >= 0 ? m_run[i] : -INFINITY;
        row[dv + 1] = failed ? NAN : l_run[i];
      }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = g + 8 * i;
    if (r >= nh) continue;
    float f = (l_run[i] > 0.f && !failed && s_mine >= 0) ? 1.f / l_run[i] : 0.f;
    if (gate != nullptr) f *= 1.f / (1.f + expf(-__bfloat162float(gate[(size_t)t * ldg + h0 + r])));
    __nv_bfloat16* dst = out + ((size_t)t * heads + h0 + r) * dv + w4 * (dv / 4);
#pragma unroll
    for (int n = 0; n < NT; ++n)
      *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * tq) = pack_bf16(o[n][2 * i] * f, o[n][2 * i + 1] * f);
  }
}

// The splits of a (token, head): out = sum_z O_z e^(m_z - m) / (sum_z l_z e^(m_z - m) + e^(sink - m)),
// times sigmoid(gate).  One block per (token, head).
template <typename TS>
__global__ void __launch_bounds__(128)
attention_latent_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, int heads, int dv,
                              int splits, const TS* __restrict__ sink, const __nv_bfloat16* __restrict__ gate,
                              int ldg) {
  pdl_trigger();      // the next kernel may be scheduled; it waits for this one before it touches data
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const int groups = (heads + 15) / 16;
  const float* base = partial + (((size_t)t * groups + h / 16) * splits) * 16 * (dv + 2) + (size_t)(h % 16) * (dv + 2);
  const size_t step = (size_t)16 * (dv + 2);
  float m = sink != nullptr ? to_float<TS>(sink[h]) : -INFINITY;
  for (int z = 0; z < splits; ++z) m = fmaxf(m, base[z * step + dv]);
  float l = sink != nullptr ? expf(to_float<TS>(sink[h]) - m) : 0.f;
  for (int z = 0; z < splits; ++z) {
    const float mz = base[z * step + dv];
    if (mz != -INFINITY) l += base[z * step + dv + 1] * expf(mz - m);
  }
  float f = l > 0.f ? 1.f / l : 0.f;          // a NaN denominator (a bad page in some split) gives zeros
  if (gate != nullptr) f *= 1.f / (1.f + expf(-__bfloat162float(gate[(size_t)t * ldg + h])));
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    float acc = 0.f;
    for (int z = 0; z < splits; ++z) {
      const float mz = base[z * step + dv];
      if (mz != -INFINITY) acc += base[z * step + c] * expf(mz - m);
    }
    out[((size_t)t * heads + h) * dv + c] = __float2bfloat16_rn(acc * f);
  }
}

}  // namespace leone

using namespace leone;

// Returns kRefusedSize for sizes this kernel does not take (the caller asks `..._supported` first).
extern "C" int leone_attention_latent_mma_supported(int dk, int dv) {
  const int nt = dv / 32;
  return dk % 16 == 0 && dv % 32 == 0 && dv <= dk && dk <= 1024 &&
         (nt == 2 || nt == 4 || nt == 6 || nt == 8 || nt == 12 || nt == 16);
}

extern "C" int leone_attention_latent_mma(const void* q, void* out, const void* pool, const int* block_table,
                                          int table_width, const int* seq_of_token, const int* positions,
                                          int n_tokens, int heads, int dk, int dv, float scale, int window,
                                          const void* sink, int sink_dtype, const void* gate, int ldg,
                                          int page_tokens, int num_pages, int n_seqs, int splits, float* partial,
                                          int tokens_per_block, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (!leone_attention_latent_mma_supported(dk, dv) || heads <= 0 || page_tokens <= 0 || table_width <= 0 ||
      splits < 1 || splits > 64 || (splits > 1 && partial == nullptr))
    return kRefusedSize;
  if ((heads + 15) / 16 > 65535) return kRefusedSize;
  const int pitch = dk * 2 + 16;
  const size_t group_bytes = (size_t)16 * pitch + 16 * (kTile * 2 + 16) + 128 * sizeof(float);
  // prompt portions: four tokens a block share every key tile (if the shared memory holds four groups)
  int group = (splits == 1 && n_tokens >= 64 && (size_t)kTile * pitch + 4 * group_bytes <= 220 * 1024) ? 4 : 1;
  if (tokens_per_block == 1) group = 1;
  const dim3 grid((n_tokens + group - 1) / group, (heads + 15) / 16, splits);
  const size_t smem = (size_t)kTile * pitch + group * group_bytes;
#define LAUNCH_G(TS, N, GG)                                                                                   \
  do {                                                                                                        \
    auto kern = attention_latent_mma_kernel<TS, N, GG>;                                                       \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                       \
    launch_kernel(kern, grid, dim3(kMmaThreads * GG), smem, stream, (const __nv_bfloat16*)q, (__nv_bfloat16*)out,              \
                                                   (const __nv_bfloat16*)pool, block_table, table_width,     \
                                                   seq_of_token, positions, n_tokens, heads, dk, scale,      \
                                                   window, (const TS*)sink, (const __nv_bfloat16*)gate, ldg, \
                                                   page_tokens, num_pages, n_seqs, splits, partial, status); \
  } while (0)
#define LAUNCH(TS, N)                   \
  do {                                  \
    if (group == 4) LAUNCH_G(TS, N, 4); \
    else LAUNCH_G(TS, N, 1);            \
  } while (0)
#define BY_NT(TS)                       \
  switch (dv / 32) {                    \
    case 2: LAUNCH(TS, 2); break;       \
    case 4: LAUNCH(TS, 4); break;       \
    case 6: LAUNCH(TS, 6); break;       \
    case 8: LAUNCH(TS, 8); break;       \
    case 12: LAUNCH(TS, 12); break;     \
    default: LAUNCH(TS, 16); break;     \
  }
  if (sink_dtype == 0) BY_NT(float)
  else if (sink_dtype == 1) BY_NT(__nv_bfloat16)
  else return kRefusedDtype;
#undef BY_NT
#undef LAUNCH
#undef LAUNCH_G
  if (splits > 1) {
    const dim3 mgrid(n_tokens, heads);
    if (sink_dtype == 0)
      launch_kernel(attention_latent_merge_kernel<float>, mgrid, dim3(128), 0, stream, partial, (__nv_bfloat16*)out, heads, dv, splits,
                                                                      (const float*)sink, (const __nv_bfloat16*)gate, ldg);
    else
      launch_kernel(attention_latent_merge_kernel<__nv_bfloat16>, mgrid, dim3(128), 0, stream, 
          partial, (__nv_bfloat16*)out, heads, dv, splits, (const __nv_bfloat16*)sink, (const __nv_bfloat16*)gate, ldg);
  }
  return launch_result();
}
