// bfloat16 attention with several score maps per head over the paged cache, on the tensor cores, compiled for one
// pair of sizes (-DTLLM_HEAD_DIM=<key size> -DTLLM_VALUE_DIM=<value size>, multiples of 16 up to 256).
//
// A query head has `maps` score maps, each an attention of its own (own queries, own keys) over the SAME values.
// Query rows of a token lie [head][map][KD], key rows in the cache [key/value head][map][KD], value rows
// [key/value head][VD].  A CTA serves one (request, key row) and a tile of 64 "rows"; a row is a (new token, query
// head of the group) pair, so the heads that share a key row share every key and value tile the CTA loads.  Four
// warps own 16 rows each and walk the keys together in tiles of 64, gathered from their pages with cp.async, two
// stages deep.  S = Q K^T and O += P V run on mma.sync.m16n8k16 with 32-bit accumulators.
//
// Scores, the running softmax (max, sum, rescale; exp2 on scores scaled by scale * log2 e) and the weights P stay
// 32-bit: P enters the P V product as the sum of two bfloat16 numbers, P = hi + lo with hi = bf16(P) and
// lo = bf16(P - hi), so the product sees 16 bits of every weight's mantissa (relative error 2^-17, the size of the
// 32-bit rounding of the sums themselves) where a single bfloat16 operand would keep 8.  The output rows are float32
// [token][head][map][VD], for the kernel that combines a head's maps.
//
// With a sink (a learned score per head) the softmax's denominator also holds exp(sink); it has no value row.
//
// Visibility: key j is visible to the row of a token at position p iff j <= p, j > p - window when there is a
// window, and j >= (p / chunk) * chunk when keys are visible inside a chunk of positions only.
#include "attention_tiles.cuh"

#ifndef TLLM_VALUE_DIM
#error "compile with -DTLLM_VALUE_DIM=<multiple of 16 up to 256>"
#endif

TLLM_DEFINE_LAST_ERROR

namespace tllm {

constexpr int KD = HD;                 // key size: what attention_tiles.cuh calls the head size
constexpr int VD = TLLM_VALUE_DIM;
static_assert(VD % 16 == 0 && VD >= 16 && VD <= 256, "value size must be a multiple of 16 up to 256");
constexpr int LDK = KD + 8, LDV = VD + 8;   // shared-memory row strides in elements (+16 bytes: conflict-free ldmatrix)
constexpr int BM = 64;                      // rows per CTA

struct MapsParams {
  const __nv_bfloat16* q;        // rows of q_row_stride elements; queries first in each row
  const __nv_bfloat16* kcache;   // [pages, nkv * maps, page_size, KD]
  const __nv_bfloat16* vcache;   // [pages, nkv, page_size, VD]
  const int* block_table;        // [R, max_blocks]
  const int* cu_q;               // [R + 1]
  const int* q_start;            // [R]: position of the request's first token in this step
  float* out;                    // [T, nq * maps, VD]
  const float* sink;             // [nq] or null: exp(sink) joins the denominator of every softmax of the head
  long long k_page_stride, k_head_stride, v_page_stride, v_head_stride;
  int q_row_stride, max_blocks, nq, nkv, maps, page_size, window, chunk, tiles_per_req, n_requests;
  float scale_log2;              // scale * log2(e)
  // Key tiles in `splits` runs (blockIdx.y), for steps of decoded tokens whose grid would not fill the SMs: a run
  // leaves its rows' unnormalised sums, maximum and denominator in part[run][row][VD + 2]; a second kernel joins them.
  int splits, total_rows;
  float* part;
};

__device__ __forceinline__ int lowest_key(const MapsParams& p, int pos) {
  int lo = p.window > 0 ? pos - p.window + 1 : 0;
  if (p.chunk > 0) lo = max(lo, (pos / p.chunk) * p.chunk);
  return max(lo, 0);
}

// One tile: 64 key rows of KD values and 64 value rows of VD values.  Thread t looks up the page of one row (0..63
// keys, 64..127 values); the copies are then issued so that consecutive lanes fetch consecutive 16-byte pieces of a
// row, the row's address coming from its lane by shuffle.  Rows outside [j_begin, j_end] or without a page are
// zero-filled (a value row that was never written must not reach the product: 0 x NaN).
__device__ __forceinline__ void load_tile(__nv_bfloat16* k_dst, __nv_bfloat16* v_dst, const PageLookup& pages, int j0,
                                          int j_begin, int j_end, int kh, int vh, const MapsParams& p, int tid) {
  const int warp = tid >> 5, lane = tid & 31;
  const bool is_v = warp >= 2;                 // warp-uniform
  const int row = (warp & 1) * 32 + lane;      // the key or value row of this lane
  const int j = j0 + row;
  bool ok = j >= j_begin && j <= j_end;
  const int page = ok ? pages(j / p.page_size) : -1;
  ok = ok && page >= 0;
  const __nv_bfloat16* src = is_v ? p.vcache : p.kcache;
  if (ok)
    src += is_v ? (long long)page * p.v_page_stride + (long long)vh * p.v_head_stride + (long long)(j % p.page_size) * VD
                : (long long)page * p.k_page_stride + (long long)kh * p.k_head_stride + (long long)(j % p.page_size) * KD;
  if (!is_v) {
    constexpr int C = KD / 8;
    __nv_bfloat16* dst = k_dst + (warp & 1) * 32 * LDK;
#pragma unroll
    for (int idx = lane; idx < 32 * C; idx += 32) {
      const int r = idx / C, c = idx % C;
      const unsigned long long a = __shfl_sync(0xffffffffu, (unsigned long long)src, r);
      const int okr = __shfl_sync(0xffffffffu, (int)ok, r);
      cp_async16(dst + r * LDK + c * 8, reinterpret_cast<const __nv_bfloat16*>(a) + (okr ? c * 8 : 0), okr != 0);
    }
  } else {
    constexpr int C = VD / 8;
    __nv_bfloat16* dst = v_dst + (warp & 1) * 32 * LDV;
#pragma unroll
    for (int idx = lane; idx < 32 * C; idx += 32) {
      const int r = idx / C, c = idx % C;
      const unsigned long long a = __shfl_sync(0xffffffffu, (unsigned long long)src, r);
      const int okr = __shfl_sync(0xffffffffu, (int)ok, r);
      cp_async16(dst + r * LDV + c * 8, reinterpret_cast<const __nv_bfloat16*>(a) + (okr ? c * 8 : 0), okr != 0);
    }
  }
}

template <int STAGES>
__global__ void __launch_bounds__(128, (VD <= 128 ? 3 : 1))
attention_maps_kernel(const MapsParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* k_s = q_s + BM * LDK;                 // STAGES tiles
  __nv_bfloat16* v_s = k_s + STAGES * BN * LDK;        // STAGES tiles
  int* page_slots = reinterpret_cast<int*>(v_s + STAGES * BN * LDV);
  pdl_trigger();
  pdl_wait();

  // the tiles of the latest tokens see the most keys: they start first
  const int nk = p.nkv * p.maps;
  const int kh = blockIdx.x % nk;
  const int req = (blockIdx.x / nk) % p.n_requests;
  const int tile = p.tiles_per_req - 1 - blockIdx.x / (nk * p.n_requests);
  const int kvh = kh / p.maps, map = kh % p.maps;
  const int group = p.nq / p.nkv;
  const int tok0 = p.cu_q[req];
  const int q_len = p.cu_q[req + 1] - tok0;
  const int rows_total = q_len * group;
  const int row0 = tile * BM;
  if (row0 >= rows_total) return;
  const int start = p.q_start[req];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int* table = p.block_table + (size_t)req * p.max_blocks;

  // keys this tile of rows can see at all (whole 64-key tiles)
  const int tok_lo = row0 / group;
  const int tok_hi = min(q_len - 1, (row0 + BM - 1) / group);
  const int key_hi = start + tok_hi;
  const int key_lo = lowest_key(p, start + tok_lo);    // lowest_key grows with the position
  int t_begin = key_lo / BN, t_end = key_hi / BN + 1;   // t_end exclusive
  if (p.splits > 1) {   // this CTA's run of the tiles (possibly empty: its rows then say so with a maximum of -inf)
    const int per = (t_end - t_begin + p.splits - 1) / p.splits;
    t_begin = min(t_end, t_begin + (int)blockIdx.y * per);
    t_end = min(t_end, t_begin + per);
  }
  const PageLookup pages = stage_pages(table, page_slots, t_begin * BN, t_end * BN, p.page_size, p.max_blocks, threadIdx.x, 128);
  __syncthreads();

  // ---- Q tile: row r -> token r / group, query row ((kvh * group + r % group) * maps + map)
  for (int idx = threadIdx.x; idx < BM * (KD / 8); idx += 128) {
    const int r = idx / (KD / 8), c = idx % (KD / 8);
    const int row = row0 + r;
    const bool ok = row < rows_total;
    const __nv_bfloat16* src = p.q;
    if (ok)
      src = p.q + (size_t)(tok0 + row / group) * p.q_row_stride + (size_t)((kvh * group + row % group) * p.maps + map) * KD + c * 8;
    cp_async16(q_s + r * LDK + c * 8, src, ok);
  }
  cp_async_commit();
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (t_begin + st < t_end)
      load_tile(k_s + st * BN * LDK, v_s + st * BN * LDV, pages, (t_begin + st) * BN, key_lo, key_hi, kh, kvh, p, threadIdx.x);
    cp_async_commit();
  }

  // per-thread rows: g and g + 8 of the warp's 16
  const int wrow = row0 + warp * 16;
  const bool warp_live = wrow < rows_total;   // a warp without rows (few decoded tokens) only helps to load
  const int r_a = wrow + g, r_b = r_a + 8;
  const int pos_a = start + r_a / group, pos_b = start + r_b / group;
  const bool live_a = r_a < rows_total, live_b = r_b < rows_total;
  const int lo_a = lowest_key(p, pos_a), lo_b = lowest_key(p, pos_b);
  // what all 16 rows of this warp can see (the same for every lane)
  const int warp_pos_min = start + wrow / group;
  const int warp_pos_max = start + min(rows_total - 1, wrow + 15) / group;
  const int warp_lo_max = lowest_key(p, warp_pos_max);
  const int warp_lo_min = lowest_key(p, warp_pos_min);

  float m_a = -CUDART_INF_F, m_b = -CUDART_INF_F, l_a = 0.f, l_b = 0.f;
  float o[VD / 8][4];
#pragma unroll
  for (int i = 0; i < VD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

  for (int tix = t_begin; tix < t_end; ++tix) {
    const int stage = (tix - t_begin) % STAGES;
    const __nv_bfloat16* kt = k_s + stage * BN * LDK;
    const __nv_bfloat16* vt = v_s + stage * BN * LDV;
    cp_async_wait<STAGES - 2>();   // this tile (and the queries) have landed
    __syncthreads();               // ... for every thread, and the stage read last iteration is free
    {
      const int nxt = tix + STAGES - 1;
      if (nxt < t_end) {
        const int ns = (nxt - t_begin) % STAGES;
        load_tile(k_s + ns * BN * LDK, v_s + ns * BN * LDV, pages, nxt * BN, key_lo, key_hi, kh, kvh, p, threadIdx.x);
      }
      cp_async_commit();
    }
    const int j_base = tix * BN;
    // a tile none of the warp's rows can see (behind their chunk or window, or ahead of them) is not computed
    if (!warp_live || j_base > warp_pos_max || j_base + BN - 1 < warp_lo_min) continue;

    // ---- S = Q K^T for this warp's 16 rows x 64 keys
    float s[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
    for (int k0 = 0; k0 < KD; k0 += 16) {
      uint32_t a[4];
      ldmatrix_x4(a, q_s + (warp * 16 + (lane & 15)) * LDK + k0 + (lane >> 4) * 8);
#pragma unroll
      for (int n0 = 0; n0 < BN; n0 += 16) {
        uint32_t b[4];
        ldmatrix_x4(b, kt + (n0 + (lane & 7) + (lane >> 4) * 8) * LDK + k0 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[n0 / 8], a, b[0], b[1]);
        mma_bf16(s[n0 / 8 + 1], a, b[2], b[3]);
      }
    }

    // ---- mask, running softmax in 32-bit; a tile that every row of the warp sees whole skips the mask
    const float c = p.scale_log2;
    if (!(j_base + BN - 1 <= warp_pos_min && j_base >= warp_lo_max)) {
#pragma unroll
      for (int i = 0; i < BN / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = j_base + i * 8 + t4 * 2 + e;
          if (!(live_a && j <= pos_a && j >= lo_a)) s[i][e] = -CUDART_INF_F;
          if (!(live_b && j <= pos_b && j >= lo_b)) s[i][2 + e] = -CUDART_INF_F;
        }
      }
    }
    float mx_a = -CUDART_INF_F, mx_b = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) {
      mx_a = fmaxf(mx_a, fmaxf(s[i][0], s[i][1]));
      mx_b = fmaxf(mx_b, fmaxf(s[i][2], s[i][3]));
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float mn_a = fmaxf(m_a, mx_a * c), mn_b = fmaxf(m_b, mx_b * c);   // running maxima in scaled units
    const float ms_a = mn_a == -CUDART_INF_F ? 0.f : mn_a, ms_b = mn_b == -CUDART_INF_F ? 0.f : mn_b;
    const float corr_a = ex2(m_a - ms_a), corr_b = ex2(m_b - ms_b);   // 0 while nothing was seen
    m_a = mn_a; m_b = mn_b;
    float sum_a = 0.f, sum_b = 0.f;
    uint32_t p_hi[BN / 16][4], p_lo[BN / 16][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) {
      const float p0 = ex2(fmaf(s[i][0], c, -ms_a)), p1 = ex2(fmaf(s[i][1], c, -ms_a));
      const float p2 = ex2(fmaf(s[i][2], c, -ms_b)), p3 = ex2(fmaf(s[i][3], c, -ms_b));
      sum_a += p0 + p1;
      sum_b += p2 + p3;
      // accumulator layout of two adjacent 8-key tiles = A-operand layout of one 16-key step
      const __nv_bfloat162 h01 = __floats2bfloat162_rn(p0, p1), h23 = __floats2bfloat162_rn(p2, p3);
      const float2 f01 = __bfloat1622float2(h01), f23 = __bfloat1622float2(h23);
      p_hi[i / 2][(i & 1) * 2 + 0] = *reinterpret_cast<const uint32_t*>(&h01);
      p_hi[i / 2][(i & 1) * 2 + 1] = *reinterpret_cast<const uint32_t*>(&h23);
      p_lo[i / 2][(i & 1) * 2 + 0] = pack_bf16(p0 - f01.x, p1 - f01.y);
      p_lo[i / 2][(i & 1) * 2 + 1] = pack_bf16(p2 - f23.x, p3 - f23.y);
    }
    l_a = l_a * corr_a + sum_a;   // per-thread partial sums; reduced across the quad at the end
    l_b = l_b * corr_b + sum_b;
#pragma unroll
    for (int i = 0; i < VD / 8; ++i) { o[i][0] *= corr_a; o[i][1] *= corr_a; o[i][2] *= corr_b; o[i][3] *= corr_b; }

    // ---- O += (P_hi + P_lo) V
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
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
  }
  cp_async_wait<0>();
  if (!warp_live) return;

  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);

  // ---- write: rows -> (token, head, map)
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = half ? r_b : r_a;
    if (row >= rows_total) continue;
    if (p.splits > 1) {
      const size_t rid = (size_t)(tok0 + row / group) * p.nq * p.maps + (size_t)((kvh * group + row % group) * p.maps + map);
      float* dst = p.part + ((size_t)blockIdx.y * p.total_rows + rid) * (VD + 2);
#pragma unroll
      for (int i = 0; i < VD / 8; ++i)
        *reinterpret_cast<float2*>(dst + i * 8 + t4 * 2) = make_float2(o[i][half * 2], o[i][half * 2 + 1]);
      if (t4 == 0) { dst[VD] = half ? m_b : m_a; dst[VD + 1] = half ? l_b : l_a; }
      continue;
    }
    float inv = 1.f / (half ? l_b : l_a);
    if (p.sink != nullptr) {   // both terms of the denominator against the larger of the running maximum and the sink
      const float sk = p.sink[kvh * group + row % group] * 1.4426950408889634f, m = half ? m_b : m_a;
      const float top = fmaxf(m, sk), f = ex2(m - top);
      inv = f / fmaf(half ? l_b : l_a, f, ex2(sk - top));
    }
    float* dst = p.out + ((size_t)(tok0 + row / group) * p.nq * p.maps + (size_t)((kvh * group + row % group) * p.maps + map)) * VD;
#pragma unroll
    for (int i = 0; i < VD / 8; ++i)
      *reinterpret_cast<float2*>(dst + i * 8 + t4 * 2) = make_float2(o[i][half * 2] * inv, o[i][half * 2 + 1] * inv);
  }
}

// Joins the runs of one row: with M the largest of the runs' maxima (and the sink), out = sum_s o_s 2^(m_s - M) /
// (sum_s l_s 2^(m_s - M) + 2^(sink - M)), runs in ascending order.  One warp per row.
__global__ void __launch_bounds__(128) attention_maps_merge_kernel(const float* __restrict__ part, float* __restrict__ out,
                                                                   const float* __restrict__ sink, int total_rows, int splits,
                                                                   int heads_maps, int maps) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= total_rows) return;
  constexpr int LD = VD + 2;
  float top = -CUDART_INF_F;
  for (int s = 0; s < splits; ++s) top = fmaxf(top, part[((size_t)s * total_rows + row) * LD + VD]);
  float extra = 0.f;
  if (sink != nullptr) {
    const float sk = sink[(row % heads_maps) / maps] * 1.4426950408889634f;
    top = fmaxf(top, sk);
    extra = ex2(sk - top);
  }
  float denom = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float* src = part + ((size_t)s * total_rows + row) * LD;
    denom = fmaf(src[VD + 1], ex2(src[VD] - top), denom);     // an empty run: 2^(-inf) = 0
  }
  const float inv = 1.f / (denom + extra);
  for (int d = lane; d < VD; d += 32) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float* src = part + ((size_t)s * total_rows + row) * LD;
      acc = fmaf(src[d], ex2(src[VD] - top), acc);
    }
    out[(size_t)row * VD + d] = acc * inv;
  }
}

}  // namespace tllm

using namespace tllm;

extern "C" int tllm_attention_maps_mma(const void* q, int q_row_stride, const void* kcache, const void* vcache,
                                       const int* block_table, int max_blocks, const int* cu_q, const int* q_start,
                                       float* out, int n_tokens, int n_requests, int max_q_len, int nq, int nkv, int maps,
                                       int kd, int vd, int page_size, long long k_page_stride, long long k_head_stride,
                                       long long v_page_stride, long long v_head_stride, float scale, int window, int chunk,
                                       const float* sink, int splits, float* part, void* stream) {
  TLLM_REQUIRE(splits >= 1 && splits <= 65535 && (splits == 1 || (part != nullptr && max_q_len * (nq / nkv) <= BM)),
               "attention_maps_mma: %d runs of key tiles need a buffer and rows that fit one tile", splits);
  TLLM_REQUIRE(kd == KD && vd == VD, "attention_maps_mma: built for key size %d and value size %d, called with %d and %d", KD, VD, kd, vd);
  TLLM_REQUIRE(n_tokens > 0 && n_requests > 0 && max_q_len > 0 && nq > 0 && nkv > 0 && nq % nkv == 0 && maps > 0,
               "attention_maps_mma: %d tokens, %d requests, %d heads, %d key/value heads, %d maps", n_tokens, n_requests, nq, nkv, maps);
  TLLM_REQUIRE(scale > 0.f, "attention_maps_mma: the score scale must be positive (got %g)", (double)scale);
  TLLM_REQUIRE(page_size > 0 && max_blocks > 0 && window >= 0 && chunk >= 0, "attention_maps_mma: page size %d, %d blocks, window %d, chunk %d", page_size, max_blocks, window, chunk);
  TLLM_REQUIRE(((uintptr_t)q % 16) == 0 && (q_row_stride % 8) == 0 && ((uintptr_t)kcache % 16) == 0 && ((uintptr_t)vcache % 16) == 0 &&
               (k_page_stride % 8) == 0 && (k_head_stride % 8) == 0 && (v_page_stride % 8) == 0 && (v_head_stride % 8) == 0 &&
               ((uintptr_t)out % 8) == 0, "attention_maps_mma: rows must be 16-byte aligned");
  const int group = nq / nkv;
  MapsParams p;
  p.q = (const __nv_bfloat16*)q; p.kcache = (const __nv_bfloat16*)kcache; p.vcache = (const __nv_bfloat16*)vcache;
  p.block_table = block_table; p.cu_q = cu_q; p.q_start = q_start; p.out = out; p.sink = sink;
  p.k_page_stride = k_page_stride; p.k_head_stride = k_head_stride; p.v_page_stride = v_page_stride; p.v_head_stride = v_head_stride;
  p.q_row_stride = q_row_stride; p.max_blocks = max_blocks; p.nq = nq; p.nkv = nkv; p.maps = maps; p.page_size = page_size;
  p.window = window; p.chunk = chunk; p.n_requests = n_requests;
  p.splits = splits; p.part = part; p.total_rows = n_tokens * nq * maps;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.tiles_per_req = (int)(((long long)max_q_len * group + BM - 1) / BM);
  const long long gx = (long long)n_requests * p.tiles_per_req * nkv * maps;
  TLLM_REQUIRE(gx <= 2147483647LL, "attention_maps_mma: grid too large");
  constexpr int ST = 2;
  const int smem = (BM * LDK + ST * BN * (LDK + LDV)) * 2 + TABLE_SLOTS * 4;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_maps_kernel<ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) TLLM_FAIL(TLLM_ERR_CUDA, "attention_maps_mma: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  TLLM_LAUNCH("attention_maps_mma", attention_maps_kernel<ST>, dim3((unsigned)gx, (unsigned)splits), 128, smem, (cudaStream_t)stream, p);
  if (splits > 1)
    TLLM_LAUNCH("attention_maps_merge", attention_maps_merge_kernel, dim3((unsigned)((p.total_rows + 3) / 4)), 128, 0,
                (cudaStream_t)stream, (const float*)part, out, sink, p.total_rows, splits, nq * maps, maps);
  return TLLM_OK;
}
