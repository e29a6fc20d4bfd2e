// The gated delta rule: a matrix state per head that is decayed, corrected towards the current value and read out,
//   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q            S: [key size, value size]
// with q and k unit vectors per head (q also times a constant), one decay g and one step size beta per head and
// token.  q, k and v come from short causal convolutions (one filter per channel) with SiLU behind them; the last
// taps - 1 inputs of every channel are part of the request's state, beside S.  Decays, step sizes, unit norms, the
// recurrence and the state are 32-bit; the projections are of the engine's dtype.
//
// Three variants share the kernels (`mode`):
//   0  the rule above with one decay per head and token;
//   1  a state-space recurrence without the correction, S <- g S + k (dt v)^T, o = S^T q, where the step size dt =
//      softplus(b + dt_bias) also sets the decay g = exp(-exp(A_log) dt), the convolutions have a bias, nothing is made
//      a unit vector, and the projection's channels come in the order [values | keys | queries];
//   2  the rule above with a decay per head, key channel and token, S <- diag(g) S, from a 32-bit input row of its own.
//
// delta_prepare: one warp per (token, head row).  The channels of the fused projection's row are
//   [kvh heads of queries | kvh heads of keys | heads of values | ...]; a row's channels are filtered over the
//   request's earlier tokens in this step and, ahead of them, the inputs kept in the state; SiLU; query and key rows
//   are divided by sqrt(sum(x^2) + unit_eps); the value rows' warps also leave the head's decay and step size:
//   g = exp(-exp(A_log) softplus(a + dt_bias)), beta = sigmoid(b).  All outputs float32.
// conv_state_update: the state's kept inputs after the step: the last taps - 1 of (kept inputs ++ the step's).
// delta_rule_scan: a group of 8 lanes owns one value column of one (request, head): the column's state rows lie in
//   the lanes' registers (a lane holds R consecutive rows).  Per token one round of shuffles gives the column's
//   S^T k, S^T q and k . q from the state as it was; with those
//       u = beta (v - g S^T k),   o = g S^T q + u (k . q),   S <- g S + k u
//   which is the sequence above with the read-out written in terms of the old state.  Tokens are staged in shared
//   memory eight at a time by cp.async, the next eight in flight meanwhile.  The state is kept transposed
//   ([slot, head, value column, key row]) so that a group's rows are consecutive in memory.  What is done to a state
//   element is the same sequence of operations however the request was cut into steps: the same bits.
#include "common.cuh"

TLLM_DEFINE_LAST_ERROR

namespace tllm {

__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float silu_exact(float x) { return x / (1.f + expf(-x)); }

struct PrepArgs {
  const void* proj;            // [T, ld]: channels first, then whatever else the projection carries
  int ld;
  const float* taps;           // [channels, n_taps]: the last column meets the current token
  int n_taps;
  const float* kept;           // [slots, n_taps - 1, channels]: inputs of the tokens before this step, oldest first
  const int* slots;
  const int* cu_q;
  const int* token_request;
  int heads, kv_heads, kd, vd;
  int beta_col, a_col;         // columns of the projection row that hold b and a (one per head each)
  const float* a_log;          // [heads]
  const float* dt_bias;        // [heads]
  float q_scale, unit_eps;
  float *q, *k, *v, *gb;       // [T, kv_heads * kd] x 2, [T, heads * vd], [T, heads, 2] = (decay, step size)
  int n_tokens;
  int q_c0, k_c0, v_c0;        // first channel of the queries, the keys and the values
  const float* conv_bias;      // [channels] or null
  int unit_norm;               // query and key heads are made unit vectors
  int mode;                    // see the top of the file
  const float* a_in;           // mode 2: [T, heads * kd] inputs of the decays (dt_bias has heads * kd values then)
  float* gk;                   // mode 2: [T, heads * kd] decays
};

template <typename T>
__global__ void __launch_bounds__(128) delta_prepare_kernel(PrepArgs a) {
  pdl_trigger();
  pdl_wait();
  const int units = 2 * a.kv_heads + a.heads;
  const long long task = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (task >= (long long)a.n_tokens * units) return;
  const int lane = threadIdx.x & 31;
  const int t = (int)(task / units), u = (int)(task % units);
  const int req = a.token_request[t];
  const int first = a.cu_q[req];
  const int channels = 2 * a.kv_heads * a.kd + a.heads * a.vd;
  const float* kept = a.kept + (size_t)a.slots[req] * (a.n_taps - 1) * channels;
  const T* proj = (const T*)a.proj;
  int c0, size;
  float* dst;
  const bool is_v = u >= 2 * a.kv_heads;
  if (!is_v) {
    const bool is_q = u < a.kv_heads;
    const int hh = is_q ? u : u - a.kv_heads;
    c0 = (is_q ? a.q_c0 : a.k_c0) + hh * a.kd; size = a.kd;
    dst = (is_q ? a.q : a.k) + (size_t)t * a.kv_heads * a.kd + (size_t)hh * a.kd;
  } else {
    const int h = u - 2 * a.kv_heads;
    c0 = a.v_c0 + h * a.vd; size = a.vd;
    dst = a.v + (size_t)t * a.heads * a.vd + (size_t)h * a.vd;
  }
  float ss = 0.f;
  for (int d = lane; d < size; d += 32) {
    const int c = c0 + d;
    float y = a.conv_bias ? a.conv_bias[c] : 0.f;
    for (int j = 0; j < a.n_taps; ++j) {
      const int n = t - first - (a.n_taps - 1) + j;   // index among the request's tokens of this step; < 0: kept ones
      const float x = n >= 0 ? to_f32(proj[(size_t)(first + n) * a.ld + c])
                             : kept[(size_t)(a.n_taps - 1 + n) * channels + c];
      y = fmaf(a.taps[(size_t)c * a.n_taps + j], x, y);
    }
    y = silu_exact(y);
    dst[d] = y;
    ss = fmaf(y, y, ss);
  }
  if (!is_v) {
    if (a.unit_norm) {
      ss = warp_sum(ss);
      const float f = (u < a.kv_heads ? a.q_scale : 1.f) / sqrtf(ss + a.unit_eps);
      __syncwarp();
      for (int d = lane; d < size; d += 32) dst[d] = __fmul_rn(dst[d], f);
    }
    return;
  }
  const int h = u - 2 * a.kv_heads;
  if (a.mode == 2) {
    const float rate = expf(a.a_log[h]);
    const size_t at = ((size_t)t * a.heads + h) * a.kd;
    for (int d = lane; d < a.kd; d += 32)
      a.gk[at + d] = expf(-rate * softplus_f(a.a_in[at + d] + a.dt_bias[h * a.kd + d]));
  }
  if (lane == 0) {
    const float zb = to_f32(proj[(size_t)t * a.ld + a.beta_col + h]);
    float* gb = a.gb + ((size_t)t * a.heads + h) * 2;
    if (a.mode == 1) {
      const float dt = softplus_f(zb + a.dt_bias[h]);
      gb[0] = expf(-expf(a.a_log[h]) * dt);
      gb[1] = dt;
    } else {
      gb[0] = a.mode == 2 ? 1.f : expf(-expf(a.a_log[h]) * softplus_f(to_f32(proj[(size_t)t * a.ld + a.a_col + h]) + a.dt_bias[h]));
      gb[1] = 1.f / (1.f + expf(-zb));
    }
  }
}

// One thread per (request, channel): kept[j] <- input at (the request's tokens after this step) - (n_taps - 1) + j.
// Ascending j reads only entries at or above the one it writes, so the update is done in place.
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ proj, int ld, float* __restrict__ kept_all,
                                         const int* __restrict__ slots, const int* __restrict__ cu_q, int n_taps,
                                         int channels, int n_requests) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int req = blockIdx.y;
  if (c >= channels || req >= n_requests) return;
  const int first = cu_q[req], n = cu_q[req + 1] - first;
  float* kept = kept_all + (size_t)slots[req] * (n_taps - 1) * channels;
  for (int j = 0; j < n_taps - 1; ++j) {
    const int i = n - (n_taps - 1) + j;   // index among this step's tokens; < 0: an input kept before
    kept[(size_t)j * channels + c] = i >= 0 ? to_f32(proj[(size_t)(first + i) * ld + c]) : kept[(size_t)(j + n) * channels + c];
  }
}

constexpr int DR_LANES = 8;            // lanes that share a value column
constexpr int DR_COLS = 16;            // value columns per CTA of 128 threads
constexpr int DR_TOK = 8;              // tokens staged at once

struct ScanArgs {
  const float *q, *k, *v, *gb;   // as delta_prepare leaves them
  float* state;                  // [slots, heads, vd, kd]
  const int* slots;
  const int* cu_q;
  float* out;                    // [T, heads * vd]
  int heads, kv_heads, kd, vd;
  const float* gk;               // mode 2: [T, heads * kd] decays per key channel
};

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int R, int MODE>   // R: state rows per lane, a multiple of 4: R * DR_LANES >= key size; MODE: see the top of the file
__global__ void __launch_bounds__(128) delta_rule_scan_kernel(ScanArgs a) {
  // A lane owns R consecutive state rows of its column (rows sub * R ... sub * R + R - 1), so that its part of a key
  // or query is read from shared memory in 16-byte pieces; a lane's part lies R + 4 floats from the next lane's, which
  // spreads the eight lanes of a column over all banks.
  constexpr int CH = R + 4;
  constexpr int KP = CH * DR_LANES;
  // per stage: q and k of DR_TOK tokens (rows past the key size stay zero), their values of this CTA's columns,
  // decay and step size
  __shared__ __align__(16) float sq[2][DR_TOK][KP], sk[2][DR_TOK][KP];
  __shared__ float sv[2][DR_TOK][DR_COLS], sg[2][DR_TOK][2];
  // decays per key channel: staged like q and k, except for the largest keys, whose three arrays would not fit a CTA's
  // static shared memory; those read their decays from global memory (the L1 holds a token's row for the CTA's columns)
  constexpr bool STAGED_DECAY = MODE == 2 && R < 32;
  __shared__ __align__(16) float sd[STAGED_DECAY ? 2 : 1][STAGED_DECAY ? DR_TOK : 1][STAGED_DECAY ? KP : 4];
  pdl_trigger();
  const int tid = threadIdx.x;
  const int sub = tid & (DR_LANES - 1), cl = tid / DR_LANES;
  const int h = blockIdx.y, req = blockIdx.z;
  const int col = blockIdx.x * DR_COLS + cl;
  const bool col_ok = col < a.vd;
  const int kh = h / (a.heads / a.kv_heads);
  for (int i = tid; i < 2 * DR_TOK * KP; i += 128) { (&sq[0][0][0])[i] = 0.f; (&sk[0][0][0])[i] = 0.f; }
  for (int i = tid; i < 2 * DR_TOK * DR_COLS; i += 128) (&sv[0][0][0])[i] = 0.f;
  if (STAGED_DECAY) for (int i = tid; i < 2 * DR_TOK * KP; i += 128) (&sd[0][0][0])[i] = 0.f;
  pdl_wait();
  const int t0 = a.cu_q[req], t1 = a.cu_q[req + 1];
  float* st = a.state + (((size_t)a.slots[req] * a.heads + h) * a.vd + (col_ok ? col : 0)) * a.kd;
  float s[R];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int row = sub * R + i;
    s[i] = (col_ok && row < a.kd) ? st[row] : 0.f;
  }
  __syncthreads();   // the zeros are in place before any copy lands beside them
  const int qk_ld = a.kv_heads * a.kd, v_ld = a.heads * a.vd;
  // 16-byte copies when a key row is made of whole pieces that start on 16-byte boundaries
  const bool wide = (a.kd & 3) == 0 && ((((size_t)a.q) | ((size_t)a.k) | ((size_t)a.gk)) & 15) == 0;
  const int g_ld = a.heads * a.kd;
  auto stage = [&](int buf, int tb) {
    const int nt = min(DR_TOK, t1 - tb);
    if (wide) {
      const int per = a.kd >> 2;
      for (int i = tid; i < nt * per; i += 128) {
        const int tt = i / per, d = (i - tt * per) << 2;
        const int at = (d / R) * CH + d % R;
        const size_t src = (size_t)(tb + tt) * qk_ld + (size_t)kh * a.kd + d;
        cp_async16(&sq[buf][tt][at], a.q + src);
        cp_async16(&sk[buf][tt][at], a.k + src);
        if (STAGED_DECAY) cp_async16(&sd[buf][tt][at], a.gk + (size_t)(tb + tt) * g_ld + (size_t)h * a.kd + d);
      }
    } else {
      for (int i = tid; i < nt * a.kd; i += 128) {
        const int tt = i / a.kd, d = i - tt * a.kd;
        const int at = (d / R) * CH + d % R;
        const size_t src = (size_t)(tb + tt) * qk_ld + (size_t)kh * a.kd + d;
        cp_async4(&sq[buf][tt][at], a.q + src);
        cp_async4(&sk[buf][tt][at], a.k + src);
        if (STAGED_DECAY) cp_async4(&sd[buf][tt][at], a.gk + (size_t)(tb + tt) * g_ld + (size_t)h * a.kd + d);
      }
    }
    for (int i = tid; i < nt * DR_COLS; i += 128) {
      const int tt = i / DR_COLS, c = i % DR_COLS;
      if (blockIdx.x * DR_COLS + c < a.vd)
        cp_async4(&sv[buf][tt][c], a.v + (size_t)(tb + tt) * v_ld + (size_t)h * a.vd + blockIdx.x * DR_COLS + c);
    }
    for (int i = tid; i < nt * 2; i += 128)
      cp_async4(&sg[buf][i / 2][i % 2], a.gb + ((size_t)(tb + i / 2) * a.heads + h) * 2 + i % 2);
  };
  auto fetch = [&](int buf, int tt, float* kr, float* qr) {   // this lane's part of a staged token's key and query
#pragma unroll
    for (int i = 0; i < R; i += 4) {
      const float4 kv = *reinterpret_cast<const float4*>(&sk[buf][tt][sub * CH + i]);
      const float4 qv = *reinterpret_cast<const float4*>(&sq[buf][tt][sub * CH + i]);
      kr[i] = kv.x; kr[i + 1] = kv.y; kr[i + 2] = kv.z; kr[i + 3] = kv.w;
      qr[i] = qv.x; qr[i + 1] = qv.y; qr[i + 2] = qv.z; qr[i + 3] = qv.w;
    }
  };
  stage(0, t0);
  cp_commit();
  int buf = 0;
  for (int tb = t0; tb < t1; tb += DR_TOK, buf ^= 1) {
    if (tb + DR_TOK < t1) stage(buf ^ 1, tb + DR_TOK);
    cp_commit();
    cp_wait<1>();
    __syncthreads();
    const int nt = min(DR_TOK, t1 - tb);
    float kn[R], qn[R];
    fetch(buf, 0, kn, qn);
    auto token = [&](int tt, bool more) {
      float kr[R], qr[R];
#pragma unroll
      for (int i = 0; i < R; ++i) { kr[i] = kn[i]; qr[i] = qn[i]; }
      if (more) fetch(buf, tt + 1, kn, qn);   // the next token's parts are on their way during this token's sums
      if (MODE == 2 && !STAGED_DECAY) {
        const float* gsrc = a.gk + (size_t)(tb + tt) * g_ld + (size_t)h * a.kd + sub * R;
#pragma unroll
        for (int i = 0; i < R; ++i)
          if (sub * R + i < a.kd) s[i] = __fmul_rn(s[i], __ldg(gsrc + i));
      }
      if (STAGED_DECAY) {   // the rows decay first, each by its own factor; the sums below then see the decayed state
#pragma unroll
        for (int i = 0; i < R; i += 4) {
          const float4 dv = *reinterpret_cast<const float4*>(&sd[buf][tt][sub * CH + i]);
          s[i] = __fmul_rn(s[i], dv.x); s[i + 1] = __fmul_rn(s[i + 1], dv.y);
          s[i + 2] = __fmul_rn(s[i + 2], dv.z); s[i + 3] = __fmul_rn(s[i + 3], dv.w);
        }
      }
      // four partial sums each, rows i, i + 4, i + 8, ... in one of them: short chains of dependent operations
      float pa[4] = {0.f, 0.f, 0.f, 0.f}, pb[4] = {0.f, 0.f, 0.f, 0.f}, pc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < R; ++i) {
        if (MODE != 1) pa[i & 3] = fmaf(s[i], kr[i], pa[i & 3]);
        pb[i & 3] = fmaf(s[i], qr[i], pb[i & 3]);
        pc[i & 3] = fmaf(kr[i], qr[i], pc[i & 3]);
      }
      float xa = (pa[0] + pa[1]) + (pa[2] + pa[3]);
      float xb = (pb[0] + pb[1]) + (pb[2] + pb[3]);
      float xc = (pc[0] + pc[1]) + (pc[2] + pc[3]);
#pragma unroll
      for (int o = DR_LANES / 2; o > 0; o >>= 1) {
        xa += __shfl_xor_sync(0xffffffffu, xa, o);
        xb += __shfl_xor_sync(0xffffffffu, xb, o);
        xc += __shfl_xor_sync(0xffffffffu, xc, o);
      }
      const float g = sg[buf][tt][0], beta = sg[buf][tt][1];   // mode 2: g = 1, the rows have decayed already
      const float u = MODE == 1 ? __fmul_rn(beta, sv[buf][tt][cl]) : __fmul_rn(beta, fmaf(-g, xa, sv[buf][tt][cl]));
      const float o = fmaf(u, xc, __fmul_rn(g, xb));
#pragma unroll
      for (int i = 0; i < R; ++i) s[i] = fmaf(kr[i], u, __fmul_rn(g, s[i]));
      if (sub == 0 && col_ok) a.out[(size_t)(tb + tt) * v_ld + (size_t)h * a.vd + col] = o;
    };
    if (nt == DR_TOK) {   // a whole stage: unrolled, so that loads of later tokens can move ahead of earlier sums
#pragma unroll
      for (int tt = 0; tt < DR_TOK; ++tt) token(tt, tt + 1 < DR_TOK);
    } else {
      for (int tt = 0; tt < nt; ++tt) token(tt, tt + 1 < nt);
    }
    __syncthreads();   // the stage is free for the copies after the next
  }
  cp_wait<0>();
  if (col_ok) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int row = sub * R + i;
      if (row < a.kd) st[row] = s[i];
    }
  }
}


// gated_group_norm: y = (o + D_h x) * silu(z), then y / sqrt(mean(y^2) + eps) * w over each of `parts` equal parts of a
// token's row (a part need not be a head), in 32-bit; one CTA per (token, part).  o, x float32 [T, width] (x and D
// may be absent), z rows of ldz values in the engine's dtype, w float32 [width], out [T, width] in the engine's dtype.
template <typename T>
__global__ void __launch_bounds__(128) gated_group_norm_kernel(const float* __restrict__ o, const float* __restrict__ x,
                                                               const float* __restrict__ skip, const T* __restrict__ z,
                                                               int ldz, const float* __restrict__ w, T* __restrict__ out,
                                                               int width, int parts, int vd, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const long long t = blockIdx.x / parts;
  const int part = blockIdx.x % parts, size = width / parts, c0 = part * size;
  const float* orow = o + t * width;
  const float* xrow = x ? x + t * width : nullptr;
  const T* zrow = z + t * ldz;
  auto value = [&](int c) {
    float y = orow[c];
    if (xrow) y = fmaf(skip[c / vd], xrow[c], y);
    const float g = to_f32(zrow[c]);
    return __fmul_rn(y, g / (1.f + expf(-g)));
  };
  float ss = 0.f;
  for (int i = threadIdx.x; i < size; i += blockDim.x) {
    const float y = value(c0 + i);
    ss = fmaf(y, y, ss);
  }
  ss = block_sum(ss, scratch);
  const float r = 1.f / sqrtf(ss / (float)size + eps);
  for (int i = threadIdx.x; i < size; i += blockDim.x)
    out[t * width + c0 + i] = from_f32<T>(__fmul_rn(__fmul_rn(value(c0 + i), r), w[c0 + i]));
}

}  // namespace tllm

using namespace tllm;

extern "C" int tllm_gated_group_norm(const float* o, const float* x, const float* skip, const void* z, int ldz,
                                     const float* w, void* out, long long n_tokens, int width, int parts, int vd,
                                     float eps, int dtype, void* stream) {
  TLLM_REQUIRE(n_tokens > 0 && width > 0 && parts > 0 && width % parts == 0 && vd > 0 && (x == nullptr) == (skip == nullptr),
               "gated_group_norm: %lld tokens, width %d in %d parts, heads of %d", n_tokens, width, parts, vd);
  const long long blocks = n_tokens * parts;
  TLLM_REQUIRE(blocks <= 2147483647LL, "gated_group_norm: %lld parts exceed the grid", blocks);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32)
    TLLM_LAUNCH("gated_group_norm", gated_group_norm_kernel<float>, (unsigned)blocks, 128, 0, s, o, x, skip, (const float*)z, ldz, w, (float*)out, width, parts, vd, eps);
  else if (dtype == TLLM_BF16)
    TLLM_LAUNCH("gated_group_norm", gated_group_norm_kernel<__nv_bfloat16>, (unsigned)blocks, 128, 0, s, o, x, skip, (const __nv_bfloat16*)z, ldz, w, (__nv_bfloat16*)out, width, parts, vd, eps);
  else TLLM_FAIL(TLLM_ERR_ARG, "gated_group_norm: unknown dtype code %d", dtype);
  return TLLM_OK;
}

extern "C" int tllm_delta_prepare(const void* proj, int ld, const float* taps, int n_taps, const float* kept,
                                  const int* slots, const int* cu_q, const int* token_request, int heads, int kv_heads,
                                  int kd, int vd, int beta_col, int a_col, const float* a_log, const float* dt_bias,
                                  float q_scale, float unit_eps, float* q, float* k, float* v, float* gb, int n_tokens,
                                  int q_c0, int k_c0, int v_c0, const float* conv_bias, int unit_norm, int mode,
                                  const float* a_in, float* gk, int dtype, void* stream) {
  TLLM_REQUIRE(n_tokens > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && kd > 0 && vd > 0 && n_taps >= 1,
               "delta_prepare: %d tokens, %d heads over %d query/key heads, sizes %d / %d, %d taps", n_tokens, heads, kv_heads, kd, vd, n_taps);
  PrepArgs a;
  a.proj = proj; a.ld = ld; a.taps = taps; a.n_taps = n_taps; a.kept = kept; a.slots = slots; a.cu_q = cu_q;
  a.token_request = token_request; a.heads = heads; a.kv_heads = kv_heads; a.kd = kd; a.vd = vd; a.beta_col = beta_col;
  a.a_col = a_col; a.a_log = a_log; a.dt_bias = dt_bias; a.q_scale = q_scale; a.unit_eps = unit_eps; a.q = q; a.k = k;
  a.v = v; a.gb = gb; a.n_tokens = n_tokens;
  TLLM_REQUIRE(mode >= 0 && mode <= 2 && (mode != 2 || (a_in && gk)), "delta_prepare: mode %d (0, 1 or 2; 2 needs the decays' inputs and outputs)", mode);
  a.q_c0 = q_c0; a.k_c0 = k_c0; a.v_c0 = v_c0; a.conv_bias = conv_bias; a.unit_norm = unit_norm; a.mode = mode; a.a_in = a_in; a.gk = gk;
  const long long tasks = (long long)n_tokens * (2 * kv_heads + heads);
  const long long blocks = (tasks + 3) / 4;
  TLLM_REQUIRE(blocks <= 2147483647LL, "delta_prepare: %lld rows exceed the grid", tasks);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32) TLLM_LAUNCH("delta_prepare", delta_prepare_kernel<float>, (unsigned)blocks, 128, 0, s, a);
  else if (dtype == TLLM_BF16) TLLM_LAUNCH("delta_prepare", delta_prepare_kernel<__nv_bfloat16>, (unsigned)blocks, 128, 0, s, a);
  else TLLM_FAIL(TLLM_ERR_ARG, "delta_prepare: unknown dtype code %d", dtype);
  return TLLM_OK;
}

extern "C" int tllm_conv_state_update(const void* proj, int ld, float* kept, const int* slots, const int* cu_q, int n_taps,
                                      int channels, int n_requests, int dtype, void* stream) {
  TLLM_REQUIRE(n_requests > 0 && channels > 0 && n_taps >= 1 && n_requests <= 65535,
               "conv_state_update: %d requests, %d channels, %d taps", n_requests, channels, n_taps);
  if (n_taps == 1) return TLLM_OK;
  const dim3 grid((channels + 127) / 128, n_requests);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TLLM_F32)
    TLLM_LAUNCH("conv_state_update", conv_state_update_kernel<float>, grid, 128, 0, s, (const float*)proj, ld, kept, slots, cu_q, n_taps, channels, n_requests);
  else if (dtype == TLLM_BF16)
    TLLM_LAUNCH("conv_state_update", conv_state_update_kernel<__nv_bfloat16>, grid, 128, 0, s, (const __nv_bfloat16*)proj, ld, kept, slots, cu_q, n_taps, channels, n_requests);
  else TLLM_FAIL(TLLM_ERR_ARG, "conv_state_update: unknown dtype code %d", dtype);
  return TLLM_OK;
}

extern "C" int tllm_delta_rule_scan(const float* q, const float* k, const float* v, const float* gb, float* state,
                                    const int* slots, const int* cu_q, float* out, int heads, int kv_heads, int kd, int vd,
                                    int n_requests, int mode, const float* gk, void* stream) {
  TLLM_REQUIRE(n_requests > 0 && n_requests <= 65535 && heads > 0 && heads <= 65535 && kv_heads > 0 && heads % kv_heads == 0,
               "delta_rule_scan: %d requests, %d heads over %d query/key heads", n_requests, heads, kv_heads);
  TLLM_REQUIRE(kd >= 1 && kd <= 256 && vd >= 1, "delta_rule_scan: key size %d (at most 256), value size %d", kd, vd);
  ScanArgs a;
  a.q = q; a.k = k; a.v = v; a.gb = gb; a.state = state; a.slots = slots; a.cu_q = cu_q; a.out = out; a.heads = heads;
  a.kv_heads = kv_heads; a.kd = kd; a.vd = vd; a.gk = gk;
  TLLM_REQUIRE(mode >= 0 && mode <= 2 && (mode == 2) == (gk != nullptr), "delta_rule_scan: mode %d (0, 1 or 2; decays per key channel with 2 only)", mode);
  const dim3 grid((vd + DR_COLS - 1) / DR_COLS, heads, n_requests);
  cudaStream_t s = (cudaStream_t)stream;
#define TLLM_SCAN(R)                                                                                         \
  do {                                                                                                       \
    if (mode == 0) TLLM_LAUNCH("delta_rule_scan", (delta_rule_scan_kernel<R, 0>), grid, 128, 0, s, a);       \
    else if (mode == 1) TLLM_LAUNCH("delta_rule_scan", (delta_rule_scan_kernel<R, 1>), grid, 128, 0, s, a);  \
    else TLLM_LAUNCH("delta_rule_scan", (delta_rule_scan_kernel<R, 2>), grid, 128, 0, s, a);                 \
  } while (0)
  if (kd <= 32) TLLM_SCAN(4);
  else if (kd <= 64) TLLM_SCAN(8);
  else if (kd <= 128) TLLM_SCAN(16);
  else TLLM_SCAN(32);
#undef TLLM_SCAN
  return TLLM_OK;
}
