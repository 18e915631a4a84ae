// Row kernels of a layer that norms what it reads AND what it adds, and short convolutions over time.
//
//   sandwich_norm  m = d                                     (one delta), or
//                  m = 1/2 (a / rms(a) u_a + b / rms(b) u_b)   (two deltas, each over its own root mean square)
//                  x += LN(m) w_post (+ row)                 LN(v) = (v - mean) / sqrt(var + eps), var = mean of squared deviations
//                  out = LN(x) w_pre                         (optional; of chosen rows when `rows` is given)
//   short_conv     y_t = [u_t +] act(bias + sum_j w[j] u_(t - taps + 1 + j)) per channel and request; the last taps - 1
//                  inputs of a request wait in its state slot; zeros before a request's start
//   poly_norm      a z / rms(z) + b z^2 / rms(z^2) + c z^3 / rms(z^3) + e, powers element by element
//
// All arithmetic is float32 in both compute types; only results that feed a matrix product are
// stored in the compute type.  Every row is reduced by one block in a fixed order, so a row's
// result does not depend on what else the step holds.
#include <math.h>

#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_norm_conv)

namespace {

constexpr int ROW_THREADS = 256;
constexpr int MAX_TAPS = 8;

struct SandwichArgs {
    float *x;                       // [n, E] the residual stream
    const float *d1, *d2;           // deltas [n, E] (d2 null: one delta; both null: none)
    const float *u1, *u2;           // unit weights of the two deltas [E]
    const float *w_post;            // [E] or null (the delta is added as it is)
    const float *row_add;           // [E] or null: one row added to every x
    const float *w_pre;             // [E] or null (no output)
    const int *rows;                // or null
    void *out;                      // [n_out, E]
    int E;
    float eps;
    // a step of one token a request: the convolution of the normed rows over time in the same kernel
    // (out = h + sum_j conv_w[j] h_(t - taps + 1 + j), the request's last taps - 1 rows of h in its slot)
    const float *conv_w;            // [taps, E] or null
    float *conv_state;
    long long conv_state_ld;
    const int *slots;
    int taps;
};

// sum over the block of two numbers at once, fixed order
__device__ __forceinline__ float2 block_sum2(float a, float b, float2 *red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    a = warp_sum(a), b = warp_sum(b);
    __syncthreads();
    if (lane == 0) red[warp] = make_float2(a, b);
    __syncthreads();
    float2 t = make_float2(0.f, 0.f);
    for (int w = 0; w < nwarps; ++w) t.x += red[w].x, t.y += red[w].y;
    return t;
}

template <typename TO, int NT>
__global__ void __launch_bounds__(NT) sandwich_norm_kernel(const SandwichArgs a) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float row[];          // E floats: m, then x
    __shared__ float2 red[32];
    constexpr int nthr = NT;
    const int E = a.E, tid = threadIdx.x;
    const int r = blockIdx.x;
    const size_t src = a.rows ? (size_t)a.rows[r] : (size_t)r;
    float *xr = a.x + src * E;
    const float invE = 1.0f / (float)E;
    const bool has_delta = a.d1 != nullptr;
    if (has_delta) {
        const float *d1 = a.d1 + src * E;
        if (a.d2 != nullptr) {
            const float *d2 = a.d2 + src * E;
            float s1 = 0.f, s2 = 0.f;
            for (int i = tid; i < E; i += nthr) {
                const float p = act_load(d1 + i), q = act_load(d2 + i);
                s1 = fmaf(p, p, s1), s2 = fmaf(q, q, s2);
            }
            const float2 ss = block_sum2(s1, s2, red);
            const float i1 = 0.5f / sqrtf(ss.x * invE + a.eps), i2 = 0.5f / sqrtf(ss.y * invE + a.eps);
            for (int i = tid; i < E; i += nthr)
                row[i] = act_load(d1 + i) * i1 * __ldg(a.u1 + i) + act_load(d2 + i) * i2 * __ldg(a.u2 + i);
        } else {
            for (int i = tid; i < E; i += nthr) row[i] = act_load(d1 + i);
        }
        float mean = 0.f, inv = 1.f;
        if (a.w_post != nullptr) {
            float s = 0.f;
            for (int i = tid; i < E; i += nthr) s += row[i];
            mean = block_sum2(s, 0.f, red).x * invE;
            float v = 0.f;
            for (int i = tid; i < E; i += nthr) {
                const float c = row[i] - mean;
                v = fmaf(c, c, v);
            }
            inv = 1.0f / sqrtf(block_sum2(v, 0.f, red).x * invE + a.eps);
        }
        for (int i = tid; i < E; i += nthr) {
            float m = row[i];
            if (a.w_post != nullptr) m = (m - mean) * inv * __ldg(a.w_post + i);
            float xv = act_load(xr + i) + m;
            if (a.row_add != nullptr) xv += __ldg(a.row_add + i);
            row[i] = xv;
            if (a.rows == nullptr) xr[i] = xv;
        }
    } else {
        for (int i = tid; i < E; i += nthr) {
            float xv = act_load(xr + i);
            if (a.row_add != nullptr) {
                xv += __ldg(a.row_add + i);
                if (a.rows == nullptr) xr[i] = xv;
            }
            row[i] = xv;
        }
    }
    if (a.w_pre == nullptr) return;
    float s = 0.f;
    for (int i = tid; i < E; i += nthr) s += row[i];
    const float mean = block_sum2(s, 0.f, red).x * invE;
    float v = 0.f;
    for (int i = tid; i < E; i += nthr) {
        const float c = row[i] - mean;
        v = fmaf(c, c, v);
    }
    const float inv = 1.0f / sqrtf(block_sum2(v, 0.f, red).x * invE + a.eps);
    TO *orow = reinterpret_cast<TO *>(a.out) + (size_t)r * E;
    if (a.conv_w == nullptr) {
        for (int i = tid; i < E; i += nthr) orow[i] = from_f32<TO>((row[i] - mean) * inv * __ldg(a.w_pre + i));
        return;
    }
    // row r is the one token of request r: the same sums in the same order as short_conv's
    const int back = a.taps - 1;
    float *st = a.conv_state + (size_t)a.slots[r] * a.conv_state_ld;
    for (int i = tid; i < E; i += nthr) {
        const float h = (row[i] - mean) * inv * __ldg(a.w_pre + i);
        float acc = 0.f, old[MAX_TAPS];
        for (int j = 0; j < back; ++j) old[j] = act_load(st + (size_t)j * E + i);       // every load before the first store
        for (int j = 0; j < back; ++j) {
            acc = fmaf(__ldg(a.conv_w + (size_t)j * E + i), old[j], acc);
            if (j > 0) st[(size_t)(j - 1) * E + i] = old[j];
        }
        if (back > 0) st[(size_t)(back - 1) * E + i] = h;
        acc = fmaf(__ldg(a.conv_w + (size_t)back * E + i), h, acc);
        orow[i] = from_f32<TO>(acc + h);
    }
}

__device__ __forceinline__ float silu_(float v) { return v / (1.0f + expf(-v)); }

// u float32 [n, ld_in] (C columns used); w float32 [taps, C] (row j weighs the input taps - 1 - j tokens back);
// state float32 rows of state_ld floats per slot, (taps - 1) x C of them used, oldest input first.
// A thread owns one channel of one token.  Tokens that reach back before the step's first token
// of their request read the slot; all of those (the first taps - 1 of the request in this step) are
// computed by the thread of the request's first token, which then writes the slot: nobody else
// touches that channel's floats there.
template <typename TO, int V> struct ConvVec;
template <typename TO> struct ConvVec<TO, 1> {
    static __device__ __forceinline__ void load(const float *p, float (&v)[1]) { v[0] = act_load(p); }
    static __device__ __forceinline__ void load_w(const float *p, float (&v)[1]) { v[0] = __ldg(p); }
    static __device__ __forceinline__ void store_f(float *p, const float (&v)[1]) { p[0] = v[0]; }
    static __device__ __forceinline__ void store(TO *p, const float (&v)[1]) { p[0] = from_f32<TO>(v[0]); }
};
template <typename TO> struct ConvVec<TO, 4> {
    static __device__ __forceinline__ void load(const float *p, float (&v)[4]) {
        const float4 t = act_load(reinterpret_cast<const float4 *>(p));
        v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
    }
    static __device__ __forceinline__ void load_w(const float *p, float (&v)[4]) {
        const float4 t = __ldg(reinterpret_cast<const float4 *>(p));
        v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
    }
    static __device__ __forceinline__ void store_f(float *p, const float (&v)[4]) { *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]); }
    static __device__ __forceinline__ void store(float *p, const float (&v)[4]) { store_f(p, v); }
    static __device__ __forceinline__ void store(__nv_bfloat16 *p, const float (&v)[4]) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
        float2 raw;
        raw.x = *reinterpret_cast<float *>(&lo), raw.y = *reinterpret_cast<float *>(&hi);
        *reinterpret_cast<float2 *>(p) = raw;
    }
};

// V channels a thread (4 when channels, strides and addresses allow 16-byte accesses); TAPS > 0: the taps at compile time
template <typename TO, int V, int TAPS>
__global__ void __launch_bounds__(256) short_conv_kernel(const float *__restrict__ u, int ld_in, const float *__restrict__ w,
                                                         const float *__restrict__ bias, float *__restrict__ state, long long state_ld,
                                                         const int *__restrict__ seq_of_token, const int *__restrict__ seq_start,
                                                         const int *__restrict__ slots, TO *__restrict__ out, int ld_out, int n, int C, int taps_rt,
                                                         int act, int residual, int tpt) {
    pdl_trigger();
    pdl_wait();
    using X = ConvVec<TO, V>;
    const int taps = TAPS > 0 ? TAPS : taps_rt;
    constexpr int MT = TAPS > 0 ? TAPS : MAX_TAPS;
    constexpr int RUN = 4;          // tokens a thread takes in a row when a step has many (tpt = RUN): an input row is then read once for RUN results
    const int per_row = C / V;
    const size_t total = (size_t)((n + tpt - 1) / tpt) * per_row;
    const int back = taps - 1;
    for (size_t it = (size_t)blockIdx.x * blockDim.x + threadIdx.x; it < total; it += (size_t)gridDim.x * blockDim.x) {
      const int tg = (int)(it / per_row), c = (int)(it - (size_t)tg * per_row) * V;
      const int tA = tg * tpt, tB = min(tA + tpt, n);
      if (TAPS > 0 && tpt == RUN && tB - tA == RUN) {
          const int sA = seq_of_token[tA];
          if (sA == seq_of_token[tA + RUN - 1] && tA - seq_start[sA] >= back) {
              // RUN tokens of one request, none of which reaches into the slot: a window of back + RUN input rows
              float in[MT - 1 + RUN][V], wj[MT][V], b[V];
#pragma unroll
              for (int e = 0; e < V; ++e) b[e] = 0.f;
              if (bias) X::load_w(bias + c, b);
#pragma unroll
              for (int r = 0; r < MT - 1 + RUN; ++r) X::load(u + (size_t)(tA - back + r) * ld_in + c, in[r]);
#pragma unroll
              for (int j = 0; j < MT; ++j) X::load_w(w + (size_t)j * C + c, wj[j]);
#pragma unroll
              for (int q = 0; q < RUN; ++q) {
                  float y[V];
#pragma unroll
                  for (int e = 0; e < V; ++e) {
                      float acc = b[e];
#pragma unroll
                      for (int j = 0; j < MT; ++j) acc = fmaf(wj[j][e], in[q + j][e], acc);
                      if (act == 1) acc = silu_(acc);
                      if (residual) acc += in[q + MT - 1][e];
                      y[e] = acc;
                  }
                  X::store(out + (size_t)(tA + q) * ld_out + c, y);
              }
              continue;
          }
      }
      for (int t = tA; t < tB; ++t) {
        const int s = seq_of_token[t];
        const int t0 = seq_start[s];
        const int i = t - t0;
        if (i > 0 && i < back) continue;
        float b[V];
#pragma unroll
        for (int e = 0; e < V; ++e) b[e] = 0.f;
        if (bias) X::load_w(bias + c, b);
        if (i >= back) {
            float in[MT][V], wj[MT][V];
#pragma unroll
            for (int j = 0; j < MT; ++j)
                if (j < taps) X::load(u + (size_t)(t - back + j) * ld_in + c, in[j]), X::load_w(w + (size_t)j * C + c, wj[j]);
            float y[V];
#pragma unroll
            for (int e = 0; e < V; ++e) {
                float acc = b[e], cur = 0.f;
#pragma unroll
                for (int j = 0; j < MT; ++j)
                    if (j < taps) cur = in[j][e], acc = fmaf(wj[j][e], cur, acc);
                if (act == 1) acc = silu_(acc);
                if (residual) acc += cur;
                y[e] = acc;
            }
            X::store(out + (size_t)t * ld_out + c, y);
            continue;
        }
        // the request's first token of this step
        const int n_s = seq_start[s + 1] - t0;
        float *st = state + (size_t)slots[s] * state_ld + c;
        float old[MT][V], wj[MT][V];
#pragma unroll
        for (int j = 0; j < MT; ++j) {
            if (j < back) X::load(st + (size_t)j * C, old[j]);
            if (j < taps) X::load_w(w + (size_t)j * C + c, wj[j]);
        }
        const int first = n_s < back ? n_s : back;
        for (int k = 0; k < first; ++k) {
            float y[V], acc[V], cur[V];
#pragma unroll
            for (int e = 0; e < V; ++e) acc[e] = b[e], cur[e] = 0.f;
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                if (j < taps) {
                    const int rel = k - back + j;
                    if (rel >= 0) {
                        X::load(u + (size_t)(t0 + rel) * ld_in + c, cur);
                    } else {
#pragma unroll
                        for (int r = 0; r < MT; ++r)
                            if (r == back + rel) {
#pragma unroll
                                for (int e = 0; e < V; ++e) cur[e] = old[r][e];
                            }
                    }
#pragma unroll
                    for (int e = 0; e < V; ++e) acc[e] = fmaf(wj[j][e], cur[e], acc[e]);
                }
            }
#pragma unroll
            for (int e = 0; e < V; ++e) {
                float a2 = acc[e];
                if (act == 1) a2 = silu_(a2);
                if (residual) a2 += cur[e];
                y[e] = a2;
            }
            X::store(out + (size_t)(t0 + k) * ld_out + c, y);
        }
#pragma unroll
        for (int r = 0; r < MT; ++r) {
            if (r < back) {
                const int rel = n_s - back + r;
                float v[V];
                if (rel >= 0) {
                    X::load(u + (size_t)(t0 + rel) * ld_in + c, v);
                } else {
#pragma unroll
                    for (int q = 0; q < MT; ++q)
                        if (q == back + rel) {
#pragma unroll
                            for (int e = 0; e < V; ++e) v[e] = old[q][e];
                        }
                }
                X::store_f(st + (size_t)r * C, v);
            }
        }
      }
    }
}

// z float32 [n, F] -> out [n, F]; coef float32 [4] = a, b, c, e
template <typename TO, int NT>
__global__ void __launch_bounds__(NT) poly_norm_kernel(const float *__restrict__ z, int ldz, const float *__restrict__ coef,
                                                                TO *__restrict__ out, int ldo, int F, float eps) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const float *zr = z + (size_t)blockIdx.x * ldz;
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    for (int i = threadIdx.x; i < F; i += NT) {
        const float v = act_load(zr + i), v2 = v * v;
        s1 += v2, s2 = fmaf(v2, v2, s2), s3 = fmaf(v2 * v2, v2, s3);
    }
    s1 = block_sum(s1, red), s2 = block_sum(s2, red), s3 = block_sum(s3, red);
    const float invF = 1.0f / (float)F;
    const float a = __ldg(coef) / sqrtf(s1 * invF + eps), b = __ldg(coef + 1) / sqrtf(s2 * invF + eps),
                c = __ldg(coef + 2) / sqrtf(s3 * invF + eps), e = __ldg(coef + 3);
    TO *orow = out + (size_t)blockIdx.x * ldo;
    for (int i = threadIdx.x; i < F; i += NT) {
        const float v = act_load(zr + i);
        orow[i] = from_f32<TO>(fmaf(v, fmaf(v, fmaf(v, c, b), a), e));
    }
}

static inline int grid_for(size_t items, int block) {
    size_t g = (items + block - 1) / block;
    return (int)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

}  // namespace

LGML_API int lgml_sandwich_norm(float *x, const float *d1, const float *d2, const float *u1, const float *u2, const float *w_post,
                                const float *row_add, const float *w_pre, const int *rows, void *out, int out_dtype, int n_out, int E, float eps,
                                const float *conv_w, float *conv_state, long long conv_state_ld, const int *slots, int taps, cudaStream_t stream) {
    LGML_REQUIRE(n_out >= 0 && E > 0, "sandwich_norm: bad sizes");
    LGML_REQUIRE(d2 == nullptr || (d1 != nullptr && u1 != nullptr && u2 != nullptr), "sandwich_norm: two deltas come with their unit weights");
    LGML_REQUIRE(w_pre == nullptr || out != nullptr, "sandwich_norm: a norm needs its output");
    LGML_REQUIRE((size_t)E * sizeof(float) <= 200 * 1024, "sandwich_norm: rows of %d floats do not fit shared memory", E);
    LGML_REQUIRE(conv_w == nullptr || (w_pre != nullptr && rows == nullptr && slots != nullptr && taps >= 1 && taps <= MAX_TAPS &&
                                       (taps == 1 || (conv_state != nullptr && conv_state_ld >= (long long)(taps - 1) * E))),
                 "sandwich_norm: the convolution in the same kernel needs a norm, all rows, the slots and a state of taps - 1 rows");
    if (n_out == 0) return 0;
    SandwichArgs a{x, d1, d2, u1, u2, w_post, row_add, w_pre, rows, out, E, eps, conv_w, conv_state, conv_state_ld, slots, taps};
    const size_t smem = (size_t)E * sizeof(float);
    // few rows (a decode step): a row's passes are latency, so more threads share it; many rows: blocks of 256 fill the SMs
    const int threads = (n_out <= 296 && E >= 1024) ? 1024 : ROW_THREADS;
#define LGML_SN(TO, NT)                                                                                                          \
    do {                                                                                                                         \
        if (smem > 48 * 1024) cudaFuncSetAttribute(sandwich_norm_kernel<TO, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        lgml_launch(sandwich_norm_kernel<TO, NT>, n_out, NT, smem, stream, a);                                                 \
    } while (0)
    if (out_dtype == LGML_F32) { if (threads == 1024) LGML_SN(float, 1024); else LGML_SN(float, ROW_THREADS); }
    else if (out_dtype == LGML_BF16) { if (threads == 1024) LGML_SN(__nv_bfloat16, 1024); else LGML_SN(__nv_bfloat16, ROW_THREADS); }
    else LGML_FAIL("sandwich_norm: unknown output type %d", out_dtype);
#undef LGML_SN
    return lgml_launch_status("sandwich_norm");
}

LGML_API int lgml_short_conv(const float *u, int ld_in, const float *w, const float *bias, float *state, long long state_ld,
                             const int *seq_of_token, const int *seq_start, const int *slots, void *out, int out_dtype, int ld_out, int n_tokens,
                             int C, int taps, int act, int residual, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && C > 0 && ld_in >= C && ld_out >= C, "short_conv: bad sizes");
    LGML_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "short_conv: 1 to %d taps, not %d", MAX_TAPS, taps);
    LGML_REQUIRE(taps == 1 || (state != nullptr && state_ld >= (long long)(taps - 1) * C), "short_conv: the state's rows do not hold taps - 1 inputs");
    if (n_tokens == 0) return 0;
    const bool vec = C % 4 == 0 && ld_in % 4 == 0 && ld_out % 4 == 0 && state_ld % 4 == 0 &&
                     ((((uintptr_t)u | (uintptr_t)w | (uintptr_t)bias | (uintptr_t)state) & 15) == 0) && (((uintptr_t)out & 15) == 0);
    const int tpt = n_tokens >= 256 ? 4 : 1;          // many tokens: a thread takes four in a row
    const int grid = grid_for((size_t)((n_tokens + tpt - 1) / tpt) * (vec ? C / 4 : C), 256);
#define LGML_SC(TO, V, T) lgml_launch(short_conv_kernel<TO, V, T>, grid, 256, 0, stream, u, ld_in, w, bias, state, state_ld, seq_of_token, seq_start, \
                                      slots, (TO *)out, ld_out, n_tokens, C, taps, act, residual, tpt)
#define LGML_SC_T(TO, V) \
    switch (taps) { case 2: LGML_SC(TO, V, 2); break; case 3: LGML_SC(TO, V, 3); break; case 4: LGML_SC(TO, V, 4); break; default: LGML_SC(TO, V, 0); }
    if (out_dtype == LGML_F32) { if (vec) { LGML_SC_T(float, 4) } else { LGML_SC_T(float, 1) } }
    else if (out_dtype == LGML_BF16) { if (vec) { LGML_SC_T(__nv_bfloat16, 4) } else { LGML_SC_T(__nv_bfloat16, 1) } }
    else LGML_FAIL("short_conv: unknown output type %d", out_dtype);
#undef LGML_SC_T
#undef LGML_SC
    return lgml_launch_status("short_conv");
}

LGML_API int lgml_poly_norm(const float *z, int ldz, const float *coef, void *out, int out_dtype, int ldo, int n_tokens, int F, float eps,
                            cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && F > 0 && ldz >= F && ldo >= F, "poly_norm: bad sizes");
    if (n_tokens == 0) return 0;
    const int threads = (n_tokens <= 296 && F >= 1024) ? 1024 : ROW_THREADS;      // few rows: more threads share a row's latency
#define LGML_PN(TO, NT) lgml_launch(poly_norm_kernel<TO, NT>, n_tokens, NT, 0, stream, z, ldz, coef, (TO *)out, ldo, F, eps)
    if (out_dtype == LGML_F32) { if (threads == 1024) LGML_PN(float, 1024); else LGML_PN(float, ROW_THREADS); }
    else if (out_dtype == LGML_BF16) { if (threads == 1024) LGML_PN(__nv_bfloat16, 1024); else LGML_PN(__nv_bfloat16, ROW_THREADS); }
    else LGML_FAIL("poly_norm: unknown output type %d", out_dtype);
#undef LGML_PN
    return lgml_launch_status("poly_norm");
}
