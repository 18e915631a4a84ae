// Mechanisms that carry something from one token of a request to the next, or add something of
// the token itself, around the mixers:
//
//   token_shift    y_t = h_t + (h_(t-1) - h_t) mu, per channel; h_(-1) = 0; the last h of a portion
//                  waits in the request's state slot for the next portion
//   mingru_scan    S_t = (1 - z_t) S_(t-1) + z_t c_t per channel, z = sigmoid(a), c = u + 1/2 (u >= 0)
//                  or sigmoid(u) (u < 0); out_t = S_t silu(g_t); S lives in the state slot
//   mingru_chunks  the same recurrence for long portions in three passes: every chunk of tokens gives
//                  (prod (1 - z), the scan from zero), the chunks' ends are chained, then every chunk
//                  runs again from its true start
//   token_side     x += m delta;  y = W_p (gelu_tanh(W_g x) e_token);  x += m y / rms(y) w
//
// Everything here is float32 arithmetic in both compute types; only the results that feed a
// matrix product (token_shift's y, the scan's out) are stored in the compute type.
#include <cooperative_groups.h>
#include <math.h>

#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_token_mix)

namespace {

__device__ __forceinline__ float sigmoidf_(float v) { return 1.0f / (1.0f + expf(-v)); }

template <typename TO> __device__ __forceinline__ void store4(TO *p, const float (&v)[4]);
template <> __device__ __forceinline__ void store4<float>(float *p, const float (&v)[4]) {
    *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16 *p, const float (&v)[4]) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    float2 raw;
    raw.x = *reinterpret_cast<float *>(&lo), raw.y = *reinterpret_cast<float *>(&hi);
    *reinterpret_cast<float2 *>(p) = raw;
}

// h float32 [n, W]; out [n, W]; state float32 rows of `state_ld` floats, one per slot, W of them used.
// A thread takes four channels of one token (one when W is no multiple of 4).  The thread of a
// request's first token of this step reads the slot and then writes the portion's last h into it:
// nobody else touches those four floats.
template <typename TO, int V>
__global__ void __launch_bounds__(256) token_shift_kernel(const float *__restrict__ h, const float *__restrict__ mu, float *__restrict__ state,
                                                          long long state_ld, const int *__restrict__ seq_of_token, const int *__restrict__ seq_start,
                                                          const int *__restrict__ slots, TO *__restrict__ out, int n, int W) {
    pdl_trigger();
    pdl_wait();
    const int per_row = W / V;
    const size_t total = (size_t)n * per_row;
    for (size_t it = (size_t)blockIdx.x * blockDim.x + threadIdx.x; it < total; it += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(it / per_row), c = (int)(it - (size_t)t * per_row) * V;
        const int s = seq_of_token[t];
        const int t0 = seq_start[s];
        float cur[4], prev[4], m[4], y[4];
        if (V == 4) {
            const float4 a = act_load(reinterpret_cast<const float4 *>(h + (size_t)t * W + c));
            cur[0] = a.x, cur[1] = a.y, cur[2] = a.z, cur[3] = a.w;
            const float4 b = __ldg(reinterpret_cast<const float4 *>(mu + c));
            m[0] = b.x, m[1] = b.y, m[2] = b.z, m[3] = b.w;
        } else {
            cur[0] = act_load(h + (size_t)t * W + c);
            m[0] = __ldg(mu + c);
        }
        if (t == t0) {
            float *st = state + (size_t)slots[s] * state_ld + c;
            const float *last = h + (size_t)(seq_start[s + 1] - 1) * W + c;
#pragma unroll
            for (int e = 0; e < V; ++e) {
                prev[e] = act_load(st + e);
                st[e] = act_load(last + e);
            }
        } else {
#pragma unroll
            for (int e = 0; e < V; ++e) prev[e] = act_load(h + (size_t)(t - 1) * W + c + e);
        }
#pragma unroll
        for (int e = 0; e < V; ++e) y[e] = fmaf(prev[e] - cur[e], m[e], cur[e]);
        if (V == 4) store4<TO>(out + (size_t)t * W + c, y);
        else out[(size_t)t * W + c] = from_f32<TO>(y[0]);
    }
}

// candidate of the recurrence: u + 1/2 where u >= 0, sigmoid(u) where u < 0 (continuous, positive)
__device__ __forceinline__ float mingru_candidate(float u) { return u >= 0.f ? u + 0.5f : sigmoidf_(u); }

// proj float32 [n, ld]: per token z-logits at column 0, u at W, g at 2 W.  A thread owns one channel of
// one request and walks its tokens in order; the loads of AHEAD tokens are in flight at a time.
template <typename TO>
__global__ void __launch_bounds__(128) mingru_scan_kernel(const float *__restrict__ proj, int ld, float *__restrict__ state, long long state_ld,
                                                          const int *__restrict__ seq_start, const int *__restrict__ slots, TO *__restrict__ out,
                                                          int W) {
    pdl_trigger();
    pdl_wait();
    constexpr int AHEAD = 8;
    const int c = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
    if (c >= W) return;
    const int t0 = seq_start[s], t1 = seq_start[s + 1];
    float *st = state + (size_t)slots[s] * state_ld + c;
    float S = act_load(st);
    for (int t = t0; t < t1; t += AHEAD) {
        float a[AHEAD], u[AHEAD], g[AHEAD];
#pragma unroll
        for (int i = 0; i < AHEAD; ++i)
            if (t + i < t1) {
                const float *row = proj + (size_t)(t + i) * ld + c;
                a[i] = act_load(row), u[i] = act_load(row + W), g[i] = act_load(row + 2 * W);
            }
#pragma unroll
        for (int i = 0; i < AHEAD; ++i)
            if (t + i < t1) {
                const float z = sigmoidf_(a[i]);
                S = fmaf(z, mingru_candidate(u[i]) - S, S);         // (1 - z) S + z c
                out[(size_t)(t + i) * W + c] = from_f32<TO>(S * g[i] * sigmoidf_(g[i]));
            }
    }
    *st = S;
}

// The three passes for long portions.  Chunks of CHUNK tokens, counted from the start of each request's
// portion; `chunk_start[s]` is the index of request s's first chunk in the (A, B) arrays.
//   pass 1: per (chunk, channel): A = prod (1 - z), B = the scan's end from S = 0
//   pass 2: per (request, channel): S at the start of every chunk (written over B), and the slot's new state
//   pass 3: per (chunk, channel): the scan from its start, out = S silu(g)
constexpr int CHUNK = 32;
__global__ void __launch_bounds__(128) mingru_chunk_ends_kernel(const float *__restrict__ proj, int ld, const int *__restrict__ chunks,
                                                                float *__restrict__ A, float *__restrict__ B, int W) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, k = blockIdx.y;
    if (c >= W) return;
    const int t0 = chunks[2 * k], t1 = chunks[2 * k + 1];
    float a = 1.f, S = 0.f;
    for (int t = t0; t < t1; t += 8) {
        float zl[8], u[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (t + i < t1) {
                const float *row = proj + (size_t)(t + i) * ld + c;
                zl[i] = act_load(row), u[i] = act_load(row + W);
            }
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (t + i < t1) {
                const float z = sigmoidf_(zl[i]);
                S = fmaf(z, mingru_candidate(u[i]) - S, S);
                a *= 1.f - z;
            }
    }
    A[(size_t)k * W + c] = a, B[(size_t)k * W + c] = S;
}

__global__ void __launch_bounds__(128) mingru_chain_kernel(const float *__restrict__ A, float *__restrict__ B, const int *__restrict__ chunk_start,
                                                           float *__restrict__ state, long long state_ld, const int *__restrict__ slots, int W) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
    if (c >= W) return;
    float *st = state + (size_t)slots[s] * state_ld + c;
    float S = act_load(st);
    const int k1 = chunk_start[s + 1];
    for (int k = chunk_start[s]; k < k1; k += 8) {          // eight chunks' pairs in flight, then the chain through them
        float a[8], b[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (k + i < k1) a[i] = act_load(A + (size_t)(k + i) * W + c), b[i] = act_load(B + (size_t)(k + i) * W + c);
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (k + i < k1) {
                B[(size_t)(k + i) * W + c] = S;             // the state this chunk starts from
                S = fmaf(a[i], S, b[i]);
            }
    }
    *st = S;
}

template <typename TO>
__global__ void __launch_bounds__(128) mingru_chunk_scan_kernel(const float *__restrict__ proj, int ld, const int *__restrict__ chunks,
                                                                const float *__restrict__ S0, TO *__restrict__ out, int W) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, k = blockIdx.y;
    if (c >= W) return;
    const int t0 = chunks[2 * k], t1 = chunks[2 * k + 1];
    float S = act_load(S0 + (size_t)k * W + c);
    for (int t = t0; t < t1; t += 8) {
        float zl[8], u[8], g[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (t + i < t1) {
                const float *row = proj + (size_t)(t + i) * ld + c;
                zl[i] = act_load(row), u[i] = act_load(row + W), g[i] = act_load(row + 2 * W);
            }
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (t + i < t1) {
                const float z = sigmoidf_(zl[i]);
                S = fmaf(z, mingru_candidate(u[i]) - S, S);
                out[(size_t)(t + i) * W + c] = from_f32<TO>(S * g[i] * sigmoidf_(g[i]));
            }
    }
}

__device__ __forceinline__ float gelu_tanh(float z) { return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }

// Sixteen bytes of a weight row as floats: 8 of bfloat16, 4 of float32.
template <typename T> struct RowVec;
template <> struct RowVec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float *p, float (&v)[4]) {
        const float4 r = __ldg(reinterpret_cast<const float4 *>(p));
        v[0] = r.x, v[1] = r.y, v[2] = r.z, v[3] = r.w;
    }
};
template <> struct RowVec<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16 *p, float (&v)[8]) {
        const uint4 r = __ldg(reinterpret_cast<const uint4 *>(p));
        const unsigned w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) v[2 * i] = __uint_as_float(w[i] << 16), v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
};

// acc + the dot product of N weights with N floats of shared memory that start on a 16-byte border
template <int N> __device__ __forceinline__ float dot_shared(const float *s, const float (&w)[N], float acc) {
#pragma unroll
    for (int i = 0; i < N; i += 4) {
        const float4 v = *reinterpret_cast<const float4 *>(s + i);
        acc = fmaf(v.x, w[i], fmaf(v.y, w[i + 1], fmaf(v.z, w[i + 2], fmaf(v.w, w[i + 3], acc))));
    }
    return acc;
}

// A cluster of `cs` blocks per token (cs = 1: a block, no cluster).  x float32 [n, W] in place; delta float32
// [parts, n, W] or null (its parts added in order, then its bias, the sum times delta_scale into x); table
// [vocab, ld_table] whose columns col0 .. col0 + dim - 1 are this layer's; wg [dim, W], wp [W, dim] in T; norm_w float32 [W].
// Every block holds the whole row of x.  The gates are dealt out over the blocks of the cluster and read back from
// their shared memory; block r then owns rows r * ceil(W / cs) .. of wp, of y and of x, and the sum of squares
// is added up over the cluster in the order of the ranks.  With few tokens in a step this is what puts the two
// matrices' bytes on many SMs instead of one per token.
// WIDE: W and dim are multiples of 16 bytes of T and both matrices start on such a border.  Then a warp
// reads a row of wg sixteen bytes a lane, two rows at a time, and `lanes` lanes (a power of two) share a row of wp,
// so that every load of a warp covers whole lines.  Otherwise element by element.
template <typename T, bool WIDE, bool CLUSTERED>
__global__ void __launch_bounds__(512) token_side_kernel(float *__restrict__ x, const float *__restrict__ delta, int n_parts, long long part_stride,
                                                         const float *__restrict__ delta_bias, float delta_scale, const int *__restrict__ token_ids,
                                                         const T *__restrict__ table, int ld_table, int col0, int vocab, const T *__restrict__ wg,
                                                         const T *__restrict__ wp, const float *__restrict__ norm_w, float eps, float out_scale,
                                                         int W, int dim, int lanes, int cs) {
    namespace cg = cooperative_groups;
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];         // x row [W], y [W], g [dim], this block's gates [dim]
    __shared__ float red[32];
    __shared__ float slice_ss;
    float *xs = sm, *ys = sm + W, *gs = sm + 2 * W, *mine_g = gs + dim;
    constexpr int V = RowVec<T>::N;
    const int t = CLUSTERED ? blockIdx.x / cs : blockIdx.x, rank = CLUSTERED ? blockIdx.x % cs : 0;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int per = (W + cs - 1) / cs, lo = min(W, rank * per), hi = min(W, lo + per);       // this block's rows
    float *xr = x + (size_t)t * W;
    for (int k = threadIdx.x; k < W; k += blockDim.x) {
        float v = act_load(xr + k);
        if (delta) {
            float d = 0.f;
            for (int p = 0; p < n_parts; ++p) d += act_load(delta + (size_t)p * part_stride + (size_t)t * W + k);
            if (delta_bias) d += __ldg(delta_bias + k);
            v = fmaf(delta_scale, d, v);
        }
        xs[k] = v;
    }
    __syncthreads();
    int id = token_ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);           // the embedding kernel has flagged such an id
    const T *e = table + (size_t)id * ld_table + col0;
    float *g_out = CLUSTERED ? mine_g : gs;
    if (WIDE) {
        for (int j = 2 * (rank * n_warps + warp); j < dim; j += 2 * n_warps * cs) {
            const bool two = j + 1 < dim;
            const T *w0 = wg + (size_t)j * W, *w1 = w0 + (two ? W : 0);
            float d0 = 0.f, d1 = 0.f;
#pragma unroll 4
            for (int k = lane * V; k < W; k += 32 * V) {
                float a[V], b[V];
                RowVec<T>::load(w0 + k, a);
                RowVec<T>::load(w1 + k, b);
                d0 = dot_shared<V>(xs + k, a, d0), d1 = dot_shared<V>(xs + k, b, d1);
            }
            d0 = warp_sum(d0), d1 = warp_sum(d1);
            if (lane == 0) {
                g_out[j] = gelu_tanh(d0) * to_f32(e[j]);
                if (two) g_out[j + 1] = gelu_tanh(d1) * to_f32(e[j + 1]);
            }
        }
    } else {
        for (int j = rank * n_warps + warp; j < dim; j += n_warps * cs) {
            const T *w = wg + (size_t)j * W;
            float dot = 0.f;
            for (int k = lane; k < W; k += 32) dot = fmaf(xs[k], to_f32(w[k]), dot);
            dot = warp_sum(dot);
            if (lane == 0) g_out[j] = gelu_tanh(dot) * to_f32(e[j]);
        }
    }
    if (CLUSTERED) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        for (int j = threadIdx.x; j < dim; j += blockDim.x) {
            const int owner = WIDE ? ((j >> 1) / n_warps) % cs : (j / n_warps) % cs;
            gs[j] = *cluster.map_shared_rank(mine_g + j, owner);
        }
    }
    __syncthreads();
    float ss = 0.f;
    if (WIDE) {
        // U row groups a warp at a time, their loads all in flight before the first product
        constexpr int U = 4;
        const int rows = 32 / lanes, sub = lane % lanes;         // rows of wp that one load of a warp covers
        const bool mine = sub * V < dim;
        for (int k0 = lo + warp * rows * U; k0 < hi; k0 += n_warps * rows * U) {
            float a[U][V], y[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int k = k0 + u * rows + lane / lanes;
                if (k < hi && mine) RowVec<T>::load(wp + (size_t)k * dim + sub * V, a[u]);
                else {
#pragma unroll
                    for (int i = 0; i < V; ++i) a[u][i] = 0.f;
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int k = k0 + u * rows + lane / lanes;
                y[u] = mine ? dot_shared<V>(gs + sub * V, a[u], 0.f) : 0.f;
                if (k < hi)
                    for (int c = (sub + lanes) * V; c < dim; c += lanes * V) {      // rows longer than 32 lanes hold at once
                        float b[V];
                        RowVec<T>::load(wp + (size_t)k * dim + c, b);
                        y[u] = dot_shared<V>(gs + c, b, y[u]);
                    }
                for (int o = lanes >> 1; o > 0; o >>= 1) y[u] += __shfl_xor_sync(0xffffffffu, y[u], o);
                if (sub == 0 && k < hi) {
                    ys[k] = y[u];
                    ss = fmaf(y[u], y[u], ss);
                }
            }
        }
    } else {
        for (int k = lo + threadIdx.x; k < hi; k += blockDim.x) {
            const T *w = wp + (size_t)k * dim;
            float y = 0.f;
            for (int j = 0; j < dim; ++j) y = fmaf(gs[j], to_f32(w[j]), y);
            ys[k] = y;
            ss = fmaf(y, y, ss);
        }
    }
    ss = block_sum(ss, red);
    if (CLUSTERED) {
        cg::cluster_group cluster = cg::this_cluster();
        if (threadIdx.x == 0) slice_ss = ss;
        cluster.sync();
        ss = 0.f;
        for (int k = 0; k < cs; ++k) ss += *cluster.map_shared_rank(&slice_ss, k);
    }
    const float inv = out_scale / sqrtf(ss / (float)W + eps);
    for (int k = lo + threadIdx.x; k < hi; k += blockDim.x) xr[k] = fmaf(ys[k] * inv, __ldg(norm_w + k), xs[k]);
    if (CLUSTERED) cg::this_cluster().sync();     // no block leaves while another may still read its gates or its sum
}

// The pieces of the same for many tokens, where the two small products run as the framework's matrix products:
//   side_fold   x += m delta, and x in the compute type for the gate product (float32: x itself serves)
//   side_gate   g = gelu_tanh(gate) e_token, in the compute type
//   side_add    x += m y / rms(y) w, y float32
template <typename TO>
__global__ void __launch_bounds__(256) side_fold_kernel(float *__restrict__ x, const float *__restrict__ delta, int n_parts, long long part_stride,
                                                        const float *__restrict__ delta_bias, float delta_scale, TO *__restrict__ xb, int n, int W) {
    pdl_trigger();
    pdl_wait();
    const size_t total = (size_t)n * W;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float v = act_load(x + i);
        if (delta) {
            float d = 0.f;
            for (int p = 0; p < n_parts; ++p) d += act_load(delta + (size_t)p * part_stride + i);
            if (delta_bias) d += __ldg(delta_bias + (i % W));
            v = fmaf(delta_scale, d, v);
            x[i] = v;
        }
        if (xb) xb[i] = from_f32<TO>(v);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) side_gate_kernel(const float *__restrict__ gate, const int *__restrict__ token_ids, const T *__restrict__ table,
                                                        int ld_table, int col0, int vocab, T *__restrict__ g, int n, int dim) {
    pdl_trigger();
    pdl_wait();
    const size_t total = (size_t)n * dim;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / dim), j = (int)(i - (size_t)t * dim);
        int id = token_ids[t];
        id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
        g[i] = from_f32<T>(gelu_tanh(act_load(gate + i)) * to_f32(table[(size_t)id * ld_table + col0 + j]));
    }
}

__global__ void __launch_bounds__(256) side_add_kernel(float *__restrict__ x, const float *__restrict__ y, const float *__restrict__ norm_w, float eps,
                                                       float out_scale, int W) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const int t = blockIdx.x;
    const float *yr = y + (size_t)t * W;
    float ss = 0.f;
    for (int k = threadIdx.x; k < W; k += blockDim.x) {
        const float v = act_load(yr + k);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float inv = out_scale / sqrtf(ss / (float)W + eps);
    float *xr = x + (size_t)t * W;
    for (int k = threadIdx.x; k < W; k += blockDim.x) xr[k] = fmaf(act_load(yr + k) * inv, __ldg(norm_w + k), act_load(xr + k));
}

static int grid_for(size_t items, int threads) {
    const size_t blocks = (items + threads - 1) / threads;
    return (int)(blocks < 148 * 16 ? (blocks ? blocks : 1) : 148 * 16);
}
}  // namespace

LGML_API int lgml_token_shift(const float *h, const float *mu, float *state, long long state_ld, const int *seq_of_token, const int *seq_start,
                              const int *slots, void *out, int out_dtype, int n_tokens, int W, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && W > 0 && state_ld >= W, "token_shift: bad sizes");
    if (n_tokens == 0) return 0;
    const bool vec = W % 4 == 0 && state_ld % 4 == 0 && ((((uintptr_t)h | (uintptr_t)mu | (uintptr_t)state) & 15) == 0) && (((uintptr_t)out & 7) == 0);
    const int grid = grid_for((size_t)n_tokens * (vec ? W / 4 : W), 256);
#define LGML_TS(TO, V) lgml_launch(token_shift_kernel<TO, V>, grid, 256, 0, stream, h, mu, state, state_ld, seq_of_token, seq_start, slots, (TO *)out, n_tokens, W)
    if (out_dtype == LGML_F32) { if (vec) LGML_TS(float, 4); else LGML_TS(float, 1); }
    else if (out_dtype == LGML_BF16) { if (vec) LGML_TS(__nv_bfloat16, 4); else LGML_TS(__nv_bfloat16, 1); }
    else LGML_FAIL("token_shift: unknown output type %d", out_dtype);
#undef LGML_TS
    return lgml_launch_status("token_shift");
}

LGML_API int lgml_mingru_scan(const float *proj, int ld, float *state, long long state_ld, const int *seq_start, const int *slots, void *out,
                              int out_dtype, int n_seqs, int W, cudaStream_t stream) {
    LGML_REQUIRE(n_seqs >= 0 && W > 0 && ld >= 3 * W && state_ld >= W, "mingru_scan: bad sizes");
    LGML_REQUIRE(n_seqs <= 65535, "mingru_scan: too many requests");
    if (n_seqs == 0) return 0;
    dim3 grid((W + 127) / 128, n_seqs);
    if (out_dtype == LGML_F32) lgml_launch(mingru_scan_kernel<float>, grid, 128, 0, stream, proj, ld, state, state_ld, seq_start, slots, (float *)out, W);
    else if (out_dtype == LGML_BF16)
        lgml_launch(mingru_scan_kernel<__nv_bfloat16>, grid, 128, 0, stream, proj, ld, state, state_ld, seq_start, slots, (__nv_bfloat16 *)out, W);
    else LGML_FAIL("mingru_scan: unknown output type %d", out_dtype);
    return lgml_launch_status("mingru_scan");
}

// chunks int32 [n_chunks, 2]: first token row and the row past the last of each chunk, the chunks of a request in a
// row; chunk_start int32 [n_seqs + 1]; ab float32 [2, n_chunks, W] scratch of the caller.
LGML_API int lgml_mingru_chunks(const float *proj, int ld, float *state, long long state_ld, const int *chunks, const int *chunk_start, int n_chunks,
                                const int *slots, float *ab, void *out, int out_dtype, int n_seqs, int W, cudaStream_t stream) {
    LGML_REQUIRE(n_seqs >= 0 && n_chunks >= 0 && W > 0 && ld >= 3 * W && state_ld >= W, "mingru_chunks: bad sizes");
    LGML_REQUIRE(n_seqs <= 65535 && n_chunks <= 65535, "mingru_chunks: too many requests or chunks");
    if (n_seqs == 0 || n_chunks == 0) return 0;
    float *A = ab, *B = ab + (size_t)n_chunks * W;
    dim3 gc((W + 127) / 128, n_chunks), gs((W + 127) / 128, n_seqs);
    lgml_launch(mingru_chunk_ends_kernel, gc, 128, 0, stream, proj, ld, chunks, A, B, W);
    lgml_launch(mingru_chain_kernel, gs, 128, 0, stream, (const float *)A, B, chunk_start, state, state_ld, slots, W);
    if (out_dtype == LGML_F32) lgml_launch(mingru_chunk_scan_kernel<float>, gc, 128, 0, stream, proj, ld, chunks, (const float *)B, (float *)out, W);
    else if (out_dtype == LGML_BF16)
        lgml_launch(mingru_chunk_scan_kernel<__nv_bfloat16>, gc, 128, 0, stream, proj, ld, chunks, (const float *)B, (__nv_bfloat16 *)out, W);
    else LGML_FAIL("mingru_chunks: unknown output type %d", out_dtype);
    return lgml_launch_status("mingru_chunks");
}

LGML_API int lgml_mingru_chunk_tokens(void) { return CHUNK; }

LGML_API int lgml_token_side(float *x, const float *delta, int n_parts, long long part_stride, const float *delta_bias, float delta_scale,
                             const int *token_ids, const void *table, int ld_table, int col0, int vocab, const void *wg, const void *wp,
                             const float *norm_w, float eps, float out_scale, int dtype, int n_tokens, int W, int dim, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && W > 0 && dim > 0 && vocab > 0 && col0 >= 0 && col0 + dim <= ld_table, "token_side: bad sizes");
    LGML_REQUIRE(delta == nullptr || n_parts >= 1, "token_side: a delta has at least one part");
    if (n_tokens == 0) return 0;
    const size_t smem = sizeof(float) * (2 * (size_t)W + 2 * (size_t)dim);
    LGML_REQUIRE(smem <= 200 * 1024, "token_side: rows of %d and %d entries do not fit shared memory", W, dim);
    // blocks per token: as many as bring a step of few tokens onto most SMs (a cluster of up to 8)
    // (float32 keeps one block: the order in which the squares are summed must not depend on what else is in the step)
    const int cs = dtype == LGML_F32 ? 1 : n_tokens <= 18 ? 8 : n_tokens <= 37 ? 4 : n_tokens <= 74 ? 2 : 1;
#define LGML_SIDE_FORM(T, WIDE, CL)                                                                                                          \
    do {                                                                                                                                     \
        auto kernel = token_side_kernel<T, WIDE, CL>;                                                                                        \
        if (smem > 48 * 1024 && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)          \
            LGML_FAIL("token_side: cannot have %zu bytes of shared memory", smem);                                                           \
        lgml_launch_cluster(kernel, n_tokens * cs, 512, smem, stream, cs, x, delta, n_parts, part_stride, delta_bias, delta_scale, token_ids, \
                            (const T *)table, ld_table, col0, vocab, (const T *)wg, (const T *)wp, norm_w, eps, out_scale, W, dim, lanes, cs); \
    } while (0)
#define LGML_SIDE(T)                                                                                                                         \
    do {                                                                                                                                     \
        constexpr int V = RowVec<T>::N;                                                                                                      \
        const bool wide = W % V == 0 && dim % V == 0 && ((uintptr_t)wg | (uintptr_t)wp) % 16 == 0;                                           \
        int lanes = 1;                                                                                                                       \
        while (lanes < 32 && lanes * V < dim) lanes *= 2;                                                                                    \
        if (wide && cs > 1) LGML_SIDE_FORM(T, true, true);                                                                                   \
        else if (wide) LGML_SIDE_FORM(T, true, false);                                                                                       \
        else if (cs > 1) LGML_SIDE_FORM(T, false, true);                                                                                     \
        else LGML_SIDE_FORM(T, false, false);                                                                                                \
    } while (0)
    if (dtype == LGML_F32) LGML_SIDE(float);
    else if (dtype == LGML_BF16) LGML_SIDE(__nv_bfloat16);
    else LGML_FAIL("token_side: unknown type %d", dtype);
#undef LGML_SIDE
#undef LGML_SIDE_FORM
    return lgml_launch_status("token_side");
}

LGML_API int lgml_side_fold(float *x, const float *delta, int n_parts, long long part_stride, const float *delta_bias, float delta_scale, void *xb,
                            int xb_dtype, int n_tokens, int W, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && W > 0, "side_fold: bad sizes");
    LGML_REQUIRE(delta == nullptr || n_parts >= 1, "side_fold: a delta has at least one part");
    if (n_tokens == 0 || (delta == nullptr && xb == nullptr)) return 0;
    const int grid = grid_for((size_t)n_tokens * W, 256);
    if (xb == nullptr || xb_dtype == LGML_F32)
        lgml_launch(side_fold_kernel<float>, grid, 256, 0, stream, x, delta, n_parts, part_stride, delta_bias, delta_scale, (float *)xb, n_tokens, W);
    else if (xb_dtype == LGML_BF16)
        lgml_launch(side_fold_kernel<__nv_bfloat16>, grid, 256, 0, stream, x, delta, n_parts, part_stride, delta_bias, delta_scale, (__nv_bfloat16 *)xb,
                    n_tokens, W);
    else LGML_FAIL("side_fold: unknown type %d", xb_dtype);
    return lgml_launch_status("side_fold");
}

LGML_API int lgml_side_gate(const float *gate, const int *token_ids, const void *table, int ld_table, int col0, int vocab, void *g, int dtype,
                            int n_tokens, int dim, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && dim > 0 && vocab > 0 && col0 >= 0 && col0 + dim <= ld_table, "side_gate: bad sizes");
    if (n_tokens == 0) return 0;
    const int grid = grid_for((size_t)n_tokens * dim, 256);
    if (dtype == LGML_F32) lgml_launch(side_gate_kernel<float>, grid, 256, 0, stream, gate, token_ids, (const float *)table, ld_table, col0, vocab, (float *)g, n_tokens, dim);
    else if (dtype == LGML_BF16)
        lgml_launch(side_gate_kernel<__nv_bfloat16>, grid, 256, 0, stream, gate, token_ids, (const __nv_bfloat16 *)table, ld_table, col0, vocab,
                    (__nv_bfloat16 *)g, n_tokens, dim);
    else LGML_FAIL("side_gate: unknown type %d", dtype);
    return lgml_launch_status("side_gate");
}

LGML_API int lgml_side_add(float *x, const float *y, const float *norm_w, float eps, float out_scale, int n_tokens, int W, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && W > 0, "side_add: bad sizes");
    if (n_tokens == 0) return 0;
    lgml_launch(side_add_kernel, n_tokens, 256, 0, stream, x, y, norm_w, eps, out_scale, W);
    return lgml_launch_status("side_add");
}
