// The attention whose heads' scores are mixed before the softmax, on the tensor cores, for bfloat16, compiled per
// (key size, value size) (-DTLLM_HEAD_DIM, -DTLLM_VALUE_DIM, multiples of 16):
//   s_g = q_g . k_kv(g);   z_h = sum_g mix[h][g] s_g;   p_h = softmax over the visible keys of z_h;   o_h = sum p_h v_kv(h).
// One CTA takes ALL heads of 16 consecutive queries of one request, a warp per head, over tiles of 32 keys of all
// key/value heads staged by cp.async (two stages where they fit).  Per tile: warp g computes S_g = Q_g K^T
// (mma.sync m16n8k16, 32-bit sums) and leaves it in shared memory; the threads then take the tile's 16 x 32 places
// between them and mix each place's scores across the heads in 32-bit (in place); warp h reads its mixed tile back in
// the accumulators' layout, masks it, keeps the running maximum and sum of its rows in 32-bit and adds P V, the weights
// as the sum of two bfloat16 numbers (16 bits of them reach the product).  `mix` holds log2(e) times the model's
// mixing matrix, so that the exponentials are powers of two.  A step of decoded tokens cuts the key tiles into runs
// that separate CTAs walk; a run leaves unnormalised sums, maximum and denominator in a 32-bit buffer that
// attention_talk_merge joins.  The end of a row (here or in the merge): optional exp(sink) in the denominator, optional
// sigmoid(gate) per head, one rounding to the output's dtype.
#include <math_constants.h>
#include "common.cuh"
#include "attention_tiles.cuh"

#ifndef TLLM_VALUE_DIM
#define TLLM_VALUE_DIM TLLM_HEAD_DIM
#endif

TLLM_DEFINE_LAST_ERROR

namespace tllm {

constexpr int KD = TLLM_HEAD_DIM;
constexpr int VD = TLLM_VALUE_DIM;
constexpr int TM = 16;             // query rows per CTA
constexpr int TN = 32;             // keys per tile
constexpr int LDK = KD + 8;        // shared-memory row strides in elements: +16 bytes keeps ldmatrix conflict-free
constexpr int LDV = VD + 8;
constexpr int LDZ = TN + 8;        // a row of scores (32-bit)

struct TalkMmaArgs {
  const __nv_bfloat16* q;      // rows of ldq values; the first heads * KD are the query heads
  int ldq;
  const __nv_bfloat16 *kcache, *vcache;
  const int* block_table;
  int max_blocks;
  const int *cu_q, *q_start;
  const float* mix;            // [heads, heads], times log2(e)
  const float* sink;           // [heads] or null
  const __nv_bfloat16* gate;   // rows of ldg values, one per head, or null
  int ldg;
  void* out;                   // [T, heads * VD]
  int out_f32;
  int heads, kv_heads, page_size;
  int page_shift;              // log2 of the page size when that is a power of two, else -1
  long long k_page_stride, k_head_stride, v_page_stride, v_head_stride;
  int window;                  // 0: every earlier key
  int stages;                  // 1 or 2 staged tiles
  int splits;                  // runs the key tiles are cut into (blockIdx.z)
  float* part;                 // splits > 1: [splits, T * heads, VD + 2]
  int total_rows;              // T * heads
};

// A tile's rows from their pages: a thread looks a key's page up once and copies its 16-byte piece of the row for every
// key/value head (the heads of a key lie a fixed stride apart).
__device__ __forceinline__ void talk_load_tile(const TalkMmaArgs& a, __nv_bfloat16* k_dst, __nv_bfloat16* v_dst, const int* table,
                                               int j0, int j_hi, int tid, int nthreads) {
  constexpr int CK = KD / 8, CV = VD / 8;
  const int G = a.kv_heads;
  for (int idx = tid; idx < TN * CK; idx += nthreads) {
    const int c = idx % CK, j = idx / CK;
    const int pos = j0 + j;
    int page = -1, off = 0;
    if (pos <= j_hi) {
      const int blk = a.page_shift >= 0 ? pos >> a.page_shift : pos / a.page_size;
      page = table[blk];
      off = pos - blk * a.page_size;
    }
    const bool ok = page >= 0;
    const __nv_bfloat16* src = ok ? a.kcache + page * a.k_page_stride + (long long)off * KD + c * 8 : a.kcache;
    __nv_bfloat16* dst = k_dst + j * LDK + c * 8;
    for (int g = 0; g < G; ++g) cp_async16(dst + g * TN * LDK, ok ? src + g * a.k_head_stride : src, ok);
  }
  for (int idx = tid; idx < TN * CV; idx += nthreads) {
    const int c = idx % CV, j = idx / CV;
    const int pos = j0 + j;
    int page = -1, off = 0;
    if (pos <= j_hi) {
      const int blk = a.page_shift >= 0 ? pos >> a.page_shift : pos / a.page_size;
      page = table[blk];
      off = pos - blk * a.page_size;
    }
    const bool ok = page >= 0;
    const __nv_bfloat16* src = ok ? a.vcache + page * a.v_page_stride + (long long)off * VD + c * 8 : a.vcache;
    __nv_bfloat16* dst = v_dst + j * LDV + c * 8;
    for (int g = 0; g < G; ++g) cp_async16(dst + g * TN * LDV, ok ? src + g * a.v_head_stride : src, ok);
  }
}

__device__ __forceinline__ float talk_sigmoid(float x) { return 1.f / (1.f + expf(-x)); }

__global__ void __launch_bounds__(512) attention_talk_mma_kernel(TalkMmaArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  pdl_trigger();
  const int H = a.heads, G = a.kv_heads;
  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int h = tid >> 5, lane = tid & 31;
  const int g8 = lane >> 2, t4 = lane & 3;
  float* zs = reinterpret_cast<float*>(smem);                              // [H][TM][LDZ]
  float* smix = zs + H * TM * LDZ;                                         // [16][16], zeros beyond the heads
  __nv_bfloat16* k_s = reinterpret_cast<__nv_bfloat16*>(smix + 256);      // [stages][G][TN][LDK]
  __nv_bfloat16* v_s = k_s + a.stages * G * TN * LDK;                      // [stages][G][TN][LDV]
  for (int i = tid; i < 256; i += nthreads) smix[i] = (i / 16 < H && i % 16 < H) ? a.mix[(i / 16) * H + i % 16] : 0.f;
  pdl_wait();
  const int r = blockIdx.y;
  const int first = a.cu_q[r], qlen = a.cu_q[r + 1] - first;
  const int i0 = blockIdx.x * TM;
  if (i0 >= qlen) return;
  const int nq = min(TM, qlen - i0);
  const int t0 = first + i0, p0 = a.q_start[r] + i0;
  const int* table = a.block_table + (size_t)r * a.max_blocks;
  const int kvh = h / (H / G);
  const int lo = a.window > 0 ? max(0, p0 - a.window + 1) : 0, hi = p0 + nq - 1;
  int t_begin = lo / TN, t_end = hi / TN + 1;
  if (a.splits > 1) {
    const int per = (t_end - t_begin + a.splits - 1) / a.splits;
    t_begin = min(t_end, t_begin + (int)blockIdx.z * per);
    t_end = min(t_end, t_begin + per);
  }
  const int stage_k = G * TN * LDK, stage_v = G * TN * LDV;
  if (t_begin < t_end) talk_load_tile(a, k_s, v_s, table, t_begin * TN, hi, tid, nthreads);
  cp_async_commit();

  // this warp's queries as the A operands of every 16-value step, straight from global memory
  uint32_t qa[KD / 16][4];
  {
    const bool live_a = g8 < nq, live_b = g8 + 8 < nq;
    const __nv_bfloat16* qa_row = a.q + (size_t)(t0 + g8) * a.ldq + (size_t)h * KD;
    const __nv_bfloat16* qb_row = a.q + (size_t)(t0 + g8 + 8) * a.ldq + (size_t)h * KD;
#pragma unroll
    for (int ks = 0; ks < KD / 16; ++ks) {
      const int k0 = ks * 16 + 2 * t4;
      qa[ks][0] = live_a ? *reinterpret_cast<const uint32_t*>(qa_row + k0) : 0u;
      qa[ks][1] = live_b ? *reinterpret_cast<const uint32_t*>(qb_row + k0) : 0u;
      qa[ks][2] = live_a ? *reinterpret_cast<const uint32_t*>(qa_row + k0 + 8) : 0u;
      qa[ks][3] = live_b ? *reinterpret_cast<const uint32_t*>(qb_row + k0 + 8) : 0u;
    }
  }
  const int pos_a = p0 + g8, pos_b = pos_a + 8;
  const bool live_a = g8 < nq, live_b = g8 + 8 < nq;
  const int lo_a = a.window > 0 ? pos_a - a.window + 1 : 0, lo_b = a.window > 0 ? pos_b - a.window + 1 : 0;
  float m_a = -CUDART_INF_F, m_b = -CUDART_INF_F, l_a = 0.f, l_b = 0.f;
  float o[VD / 8][4];
#pragma unroll
  for (int i = 0; i < VD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

  for (int tix = t_begin; tix < t_end; ++tix) {
    const int st = a.stages == 2 ? (tix - t_begin) & 1 : 0;
    const __nv_bfloat16* kt = k_s + st * stage_k + kvh * TN * LDK;
    const __nv_bfloat16* vt = v_s + st * stage_v + kvh * TN * LDV;
    cp_async_wait<0>();
    __syncthreads();   // the tile has landed for every thread; the tile before is read to its end
    if (a.stages == 2 && tix + 1 < t_end) {
      const int ns = st ^ 1;
      talk_load_tile(a, k_s + ns * stage_k, v_s + ns * stage_v, table, (tix + 1) * TN, hi, tid, nthreads);
      cp_async_commit();
    }
    // ---- S_h = Q_h K^T for 16 rows x 32 keys
    float s[TN / 8][4];
#pragma unroll
    for (int i = 0; i < TN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < KD / 16; ++ks) {
#pragma unroll
      for (int n0 = 0; n0 < TN; n0 += 16) {
        uint32_t b[4];
        ldmatrix_x4(b, kt + (n0 + (lane & 7) + (lane >> 4) * 8) * LDK + ks * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[n0 / 8], qa[ks], b[0], b[1]);
        mma_bf16(s[n0 / 8 + 1], qa[ks], b[2], b[3]);
      }
    }
    float* mine = zs + h * TM * LDZ;
#pragma unroll
    for (int i = 0; i < TN / 8; ++i) {
      *reinterpret_cast<float2*>(mine + g8 * LDZ + i * 8 + 2 * t4) = make_float2(s[i][0], s[i][1]);
      *reinterpret_cast<float2*>(mine + (g8 + 8) * LDZ + i * 8 + 2 * t4) = make_float2(s[i][2], s[i][3]);
    }
    __syncthreads();
    // ---- the heads' scores of one place (row, key) are mixed by one thread, in place
    for (int place = tid; place < TM * TN; place += nthreads) {
      float* at = zs + (place / TN) * LDZ + place % TN;
      float sg[16];
#pragma unroll
      for (int g = 0; g < 16; ++g) sg[g] = g < H ? at[g * TM * LDZ] : 0.f;
      for (int hh = 0; hh < H; ++hh) {   // the matrix row comes in four 16-byte reads that all lanes share
        const float4* mrow = reinterpret_cast<const float4*>(smix + hh * 16);
        float z = 0.f;
#pragma unroll
        for (int g4 = 0; g4 < 4; ++g4) {
          const float4 mv = mrow[g4];
          z = fmaf(mv.x, sg[4 * g4], z); z = fmaf(mv.y, sg[4 * g4 + 1], z);
          z = fmaf(mv.z, sg[4 * g4 + 2], z); z = fmaf(mv.w, sg[4 * g4 + 3], z);
        }
        at[hh * TM * LDZ] = z;
      }
    }
    __syncthreads();
    // ---- head h's mixed tile back in the accumulators' layout; mask; running softmax in 32-bit
    const int j_base = tix * TN;
    const bool whole = nq == TM && j_base + TN - 1 <= p0 && (a.window <= 0 || j_base >= p0 + TM - a.window);
#pragma unroll
    for (int i = 0; i < TN / 8; ++i) {
      const float2 za = *reinterpret_cast<const float2*>(mine + g8 * LDZ + i * 8 + 2 * t4);
      const float2 zb = *reinterpret_cast<const float2*>(mine + (g8 + 8) * LDZ + i * 8 + 2 * t4);
      const int j = j_base + i * 8 + 2 * t4;
      if (whole) {   // every row of the CTA sees every key of the tile
        s[i][0] = za.x; s[i][1] = za.y; s[i][2] = zb.x; s[i][3] = zb.y;
      } else {
        s[i][0] = (live_a && j <= pos_a && j >= lo_a) ? za.x : -CUDART_INF_F;
        s[i][1] = (live_a && j + 1 <= pos_a && j + 1 >= lo_a) ? za.y : -CUDART_INF_F;
        s[i][2] = (live_b && j <= pos_b && j >= lo_b) ? zb.x : -CUDART_INF_F;
        s[i][3] = (live_b && j + 1 <= pos_b && j + 1 >= lo_b) ? zb.y : -CUDART_INF_F;
      }
    }
    float mx_a = -CUDART_INF_F, mx_b = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < TN / 8; ++i) {
      mx_a = fmaxf(mx_a, fmaxf(s[i][0], s[i][1]));
      mx_b = fmaxf(mx_b, fmaxf(s[i][2], s[i][3]));
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
    const float ms_a = mn_a == -CUDART_INF_F ? 0.f : mn_a, ms_b = mn_b == -CUDART_INF_F ? 0.f : mn_b;
    const float corr_a = ex2(m_a - ms_a), corr_b = ex2(m_b - ms_b);   // 0 while nothing was seen
    m_a = mn_a; m_b = mn_b;
    float sum_a = 0.f, sum_b = 0.f;
    uint32_t p_hi[TN / 16][4], p_lo[TN / 16][4];
#pragma unroll
    for (int i = 0; i < TN / 8; ++i) {
      const float p0_ = ex2(s[i][0] - ms_a), p1_ = ex2(s[i][1] - ms_a);
      const float p2_ = ex2(s[i][2] - ms_b), p3_ = ex2(s[i][3] - ms_b);
      sum_a += p0_ + p1_;
      sum_b += p2_ + p3_;
      const __nv_bfloat162 h01 = __floats2bfloat162_rn(p0_, p1_), h23 = __floats2bfloat162_rn(p2_, p3_);
      const float2 f01 = __bfloat1622float2(h01), f23 = __bfloat1622float2(h23);
      p_hi[i / 2][(i & 1) * 2 + 0] = *reinterpret_cast<const uint32_t*>(&h01);
      p_hi[i / 2][(i & 1) * 2 + 1] = *reinterpret_cast<const uint32_t*>(&h23);
      p_lo[i / 2][(i & 1) * 2 + 0] = pack_bf16(p0_ - f01.x, p1_ - f01.y);
      p_lo[i / 2][(i & 1) * 2 + 1] = pack_bf16(p2_ - f23.x, p3_ - f23.y);
    }
    l_a = l_a * corr_a + sum_a;   // per-thread partial sums; reduced across the quad at the end
    l_b = l_b * corr_b + sum_b;
    if (__any_sync(0xffffffffu, corr_a != 1.f || corr_b != 1.f)) {   // most tiles leave the maxima where they were
#pragma unroll
      for (int i = 0; i < VD / 8; ++i) { o[i][0] *= corr_a; o[i][1] *= corr_a; o[i][2] *= corr_b; o[i][3] *= corr_b; }
    }
    // ---- O += (P_hi + P_lo) V
#pragma unroll
    for (int kk = 0; kk < TN / 16; ++kk) {
#pragma unroll
      for (int d0 = 0; d0 < VD; d0 += 16) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDV + d0 + (lane >> 4) * 8);
        mma_bf16(o[d0 / 8], p_hi[kk], b[0], b[1]);
        mma_bf16(o[d0 / 8 + 1], p_hi[kk], b[2], b[3]);
        mma_bf16(o[d0 / 8], p_lo[kk], b[0], b[1]);
        mma_bf16(o[d0 / 8 + 1], p_lo[kk], b[2], b[3]);
      }
    }
    if (a.stages == 1 && tix + 1 < t_end) {
      __syncthreads();   // the only stage is read to its end
      talk_load_tile(a, k_s, v_s, table, (tix + 1) * TN, hi, tid, nthreads);
      cp_async_commit();
    }
  }
  cp_async_wait<0>();
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = g8 + 8 * half;
    if (row >= nq) continue;
    const float m = half ? m_b : m_a, l = half ? l_b : l_a;
    const size_t rid = (size_t)(t0 + row) * H + h;
    if (a.splits > 1) {
      float* dst = a.part + ((size_t)blockIdx.z * a.total_rows + rid) * (VD + 2);
#pragma unroll
      for (int i = 0; i < VD / 8; ++i)
        *reinterpret_cast<float2*>(dst + i * 8 + t4 * 2) = make_float2(o[i][half * 2], o[i][half * 2 + 1]);
      if (t4 == 0) { dst[VD] = m; dst[VD + 1] = l; }
      continue;
    }
    float f = 1.f / l;
    if (a.sink != nullptr) {   // both terms of the denominator against the larger of the running maximum and the sink
      const float sk = a.sink[h] * 1.4426950408889634f;
      const float top = fmaxf(m, sk), w = ex2(m - top);
      f = w / fmaf(l, w, ex2(sk - top));
    }
    if (a.gate != nullptr) f *= talk_sigmoid(__bfloat162float(a.gate[(size_t)(t0 + row) * a.ldg + h]));
    if (a.out_f32) {
      float* dst = (float*)a.out + rid * VD;
#pragma unroll
      for (int i = 0; i < VD / 8; ++i)
        *reinterpret_cast<float2*>(dst + i * 8 + t4 * 2) = make_float2(o[i][half * 2] * f, o[i][half * 2 + 1] * f);
    } else {
      __nv_bfloat16* dst = (__nv_bfloat16*)a.out + rid * VD;
#pragma unroll
      for (int i = 0; i < VD / 8; ++i)
        *reinterpret_cast<__nv_bfloat162*>(dst + i * 8 + t4 * 2) = __floats2bfloat162_rn(o[i][half * 2] * f, o[i][half * 2 + 1] * f);
    }
  }
}

// Joins the runs of one (token, head) row: with M the largest of the runs' maxima (and the sink), out = sum_s o_s
// 2^(m_s - M) / (sum_s l_s 2^(m_s - M) + 2^(sink - M)), runs in ascending order, times sigmoid(gate).  One warp per row.
__global__ void __launch_bounds__(128) attention_talk_merge_kernel(const float* __restrict__ part, void* __restrict__ out,
                                                                   int out_f32, const float* __restrict__ sink,
                                                                   const __nv_bfloat16* __restrict__ gate, int ldg,
                                                                   int total_rows, int splits, int heads) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= total_rows) return;
  constexpr int LD = VD + 2;
  const int h = row % heads;
  float top = -CUDART_INF_F;
  for (int s = 0; s < splits; ++s) top = fmaxf(top, part[((size_t)s * total_rows + row) * LD + VD]);
  float extra = 0.f;
  if (sink != nullptr) {
    const float sk = sink[h] * 1.4426950408889634f;
    top = fmaxf(top, sk);
    extra = ex2(sk - top);
  }
  float denom = extra;
  float acc[(VD + 31) / 32];
#pragma unroll
  for (int c = 0; c < (VD + 31) / 32; ++c) acc[c] = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float* src = part + ((size_t)s * total_rows + row) * LD;
    const float m = src[VD];
    if (m == -CUDART_INF_F) continue;   // a run that saw no key of the row
    const float w = ex2(m - top);
    denom = fmaf(src[VD + 1], w, denom);
#pragma unroll
    for (int c = 0; c < (VD + 31) / 32; ++c) {
      const int d = lane + 32 * c;
      if (d < VD) acc[c] = fmaf(src[d], w, acc[c]);
    }
  }
  float f = 1.f / denom;
  if (gate != nullptr) f *= talk_sigmoid(__bfloat162float(gate[(size_t)(row / heads) * ldg + h]));
#pragma unroll
  for (int c = 0; c < (VD + 31) / 32; ++c) {
    const int d = lane + 32 * c;
    if (d < VD) {
      if (out_f32) ((float*)out)[(size_t)row * VD + d] = acc[c] * f;
      else ((__nv_bfloat16*)out)[(size_t)row * VD + d] = __float2bfloat16_rn(acc[c] * f);
    }
  }
}

inline size_t talk_mma_smem(int heads, int kv_heads, int stages) {
  return sizeof(float) * ((size_t)heads * TM * LDZ + 256) +
         sizeof(__nv_bfloat16) * (size_t)stages * kv_heads * TN * (LDK + LDV);
}

}  // namespace tllm

using namespace tllm;

// Bytes of shared memory a CTA needs with two staged tiles and with one (the caller falls back when neither fits).
extern "C" long long tllm_attention_talk_mma_smem(int heads, int kv_heads, int stages) {
  return (long long)talk_mma_smem(heads, kv_heads, stages);
}

extern "C" int tllm_attention_talk_mma(const void* q, int ldq, const void* kcache, const void* vcache, const int* block_table,
                                       int max_blocks, const int* cu_q, const int* q_start, const float* mix_log2,
                                       const float* sink, const void* gate, int ldg, void* out, int out_f32, int n_tokens,
                                       int n_requests, int max_q_len, int heads, int kv_heads, int page_size,
                                       long long k_page_stride, long long k_head_stride, long long v_page_stride,
                                       long long v_head_stride, int window, int splits, float* part, int max_stages,
                                       void* stream) {
  TLLM_REQUIRE(n_requests > 0 && n_requests <= 65535 && max_q_len > 0 && heads > 0 && heads <= 16 && kv_heads > 0 &&
               heads % kv_heads == 0 && page_size > 0 && window >= 0 && splits >= 1 && splits <= 65535 && (splits == 1 || part),
               "attention_talk_mma: %d requests, %d heads (at most 16) over %d key/value heads, %d runs", n_requests, heads, kv_heads, splits);
  TLLM_REQUIRE(ldq % 2 == 0 && ((uintptr_t)q % 4) == 0 && k_page_stride % 8 == 0 && k_head_stride % 8 == 0 && v_page_stride % 8 == 0 &&
               v_head_stride % 8 == 0 && ((uintptr_t)kcache % 16) == 0 && ((uintptr_t)vcache % 16) == 0,
               "attention_talk_mma: query rows on 4-byte and cache rows on 16-byte boundaries are needed");
  constexpr size_t LIMIT = 220 * 1024;
  int stages = max_stages >= 2 ? 2 : 1;
  if (talk_mma_smem(heads, kv_heads, 2) > LIMIT) stages = 1;
  const size_t smem = talk_mma_smem(heads, kv_heads, stages);
  TLLM_REQUIRE(smem <= LIMIT, "attention_talk_mma: %d heads over %d key/value heads of %d / %d values need %zu bytes of shared memory",
               heads, kv_heads, KD, VD, smem);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    if (cudaFuncSetAttribute(attention_talk_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      TLLM_FAIL(TLLM_ERR_CUDA, "attention_talk_mma: %zu bytes of shared memory were refused", smem);
    configured = smem;
  }
  TalkMmaArgs a;
  a.q = (const __nv_bfloat16*)q; a.ldq = ldq; a.kcache = (const __nv_bfloat16*)kcache; a.vcache = (const __nv_bfloat16*)vcache;
  a.block_table = block_table; a.max_blocks = max_blocks; a.cu_q = cu_q; a.q_start = q_start; a.mix = mix_log2; a.sink = sink;
  a.gate = (const __nv_bfloat16*)gate; a.ldg = ldg; a.out = out; a.out_f32 = out_f32; a.heads = heads; a.kv_heads = kv_heads;
  a.page_size = page_size; a.page_shift = -1;
  for (int sft = 0; sft < 31; ++sft)
    if ((1 << sft) == page_size) a.page_shift = sft;
  a.k_page_stride = k_page_stride; a.k_head_stride = k_head_stride; a.v_page_stride = v_page_stride;
  a.v_head_stride = v_head_stride; a.window = window; a.stages = stages; a.splits = splits; a.part = part;
  a.total_rows = n_tokens * heads;
  cudaStream_t s = (cudaStream_t)stream;
  const dim3 grid((max_q_len + TM - 1) / TM, n_requests, splits);
  TLLM_LAUNCH("attention_talk_mma", attention_talk_mma_kernel, grid, 32 * heads, smem, s, a);
  if (splits > 1) {
    const int rows = n_tokens * heads;
    TLLM_LAUNCH("attention_talk_merge", attention_talk_merge_kernel, (rows + 3) / 4, 128, 0, s, (const float*)part, out, out_f32,
                sink, (const __nv_bfloat16*)gate, ldg, rows, splits, heads);
  }
  return TLLM_OK;
}
