// A mixture of experts as a feed-forward: a router picks `top` of X small gated feed-forward
// layers per token; the token's output is the weighted sum of theirs.
//
//   z      = W_r h + b_r                              float32, X logits per token
//   chosen = the `top` largest z (ties: the lower index), w = softmax over the chosen z alone
//   y      = sum_e w_e W_down[e] (silu(W_gate[e] h) * (W_up[e] h))
//
// moe_router writes the chosen experts and their weights, [tokens, top] each.  The experts'
// matrices lie stacked: gate and up as [X, 2 F, E] with the gate row of a feature followed by its up row (the layout
// whose product has both in one thread's hands), down as [X, E, F].
//
// Two forms of the experts' products.  The row form (moe_gate_up, moe_down): a block per (token,
// chosen expert), a warp per output feature, k in a fixed order; it reads an expert's matrices
// once per token that chose it, which is what a decode step needs and no more, and it is the
// 32-bit path.  The grouped form for many tokens is further down.
#include <math.h>

#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_moe)

namespace {

template <typename T>
__global__ void __launch_bounds__(128) moe_router_kernel(const T *__restrict__ h, int ldh, const float *__restrict__ wr, const float *__restrict__ br,
                                                         int *__restrict__ ids, float *__restrict__ wts, int E, int X, int top, int mode,
                                                         float route_scale, int n_extra, float *__restrict__ extra) {
    pdl_trigger();
    pdl_wait();
    // X choice values (+ n_extra logits of rows that are no experts), X scores (mode 1), then the token's row (E floats, from a 16-byte boundary)
    extern __shared__ __align__(16) float rsm[];
    const int zn = (X + n_extra + 3) & ~3;
    float *z = rsm, *sc = rsm + zn, *hs = rsm + 2 * zn;
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const T *row = h + (size_t)t * ldh;
    for (int k = threadIdx.x; k < E; k += blockDim.x) hs[k] = to_f32(act_load(row + k));
    __syncthreads();
    // one order of summation whatever the batch: lane l takes elements 4 l .. 4 l + 3 of every run of 128, then the warp's tree
    const bool vec = (E % 4 == 0) && ((reinterpret_cast<uintptr_t>(wr) & 15) == 0);
    for (int e = warp; e < X + n_extra; e += n_warps) {
        const float *w = wr + (size_t)e * E;
        float dot = 0.f;
        if (vec) {
#pragma unroll 4
            for (int k = lane * 4; k < E; k += 128) {
                const float4 a = *reinterpret_cast<const float4 *>(hs + k), b = __ldg(reinterpret_cast<const float4 *>(w + k));
                dot = fmaf(a.x, b.x, fmaf(a.y, b.y, fmaf(a.z, b.z, fmaf(a.w, b.w, dot))));
            }
        } else {
            for (int k = lane; k < E; k += 32) dot = fmaf(hs[k], w[k], dot);
        }
        dot = warp_sum(dot);
        if (lane == 0) {
            if (e >= X) {
                // rows behind the experts': a gate of the token (sigmoid of its logit), for the caller
                extra[(size_t)t * n_extra + (e - X)] = 1.0f / (1.0f + expf(-dot));
            } else if (mode == 1) {
                // scores are sigmoids; the bias only corrects the choice, the weights use the plain scores
                const float sg = 1.0f / (1.0f + expf(-dot));
                sc[e] = sg;
                z[e] = sg + (br ? br[e] : 0.f);
            } else {
                z[e] = dot + (br ? br[e] : 0.f);
            }
        }
    }
    __syncthreads();
    if (warp != 0) return;
    float zmax = 0.f, sum = 0.f;
    for (int s = 0; s < top; ++s) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < X; e += 32) {
            const float v = z[e];
            if (v > best) best = v, at = e;         // strictly greater: a lane keeps its lowest index
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) best = ob, at = oa;
        }
        if (at == 0x7fffffff) at = 0;               // every logit was -inf or NaN
        if (s == 0) zmax = best;
        const float p = mode == 1 ? sc[at] : expf(best - zmax);
        sum += p;
        if (lane == 0) {
            ids[(size_t)t * top + s] = at;
            wts[(size_t)t * top + s] = p;
            z[at] = -INFINITY;
        }
        __syncwarp();
    }
    // mode 0: softmax over the chosen logits; mode 1: the chosen scores over their sum (+ 1e-20), times a constant
    const float inv = mode == 1 ? route_scale / (sum + 1e-20f) : 1.0f / sum;
    for (int s = lane; s < top; s += 32) wts[(size_t)t * top + s] *= inv;
}

// dot products of `NF` weight rows (bfloat16, 16-byte loads) with one float32 vector in shared memory: the loads of all rows of a
// step go out before any is used.  Lane l takes elements 8 l .. 8 l + 7 of every run of 256; the warp's tree adds the lanes.
template <int NF>
__device__ __forceinline__ void rows_dot_bf16(const __nv_bfloat16 *const (&rows)[NF], const float *x, int K, int lane, float (&out)[NF]) {
#pragma unroll
    for (int i = 0; i < NF; ++i) out[i] = 0.f;
    for (int k = lane * 8; k < K; k += 256) {
        uint4 raw[NF];
#pragma unroll
        for (int i = 0; i < NF; ++i) raw[i] = __ldg(reinterpret_cast<const uint4 *>(rows[i] + k));
        const float4 xa = *reinterpret_cast<const float4 *>(x + k), xb = *reinterpret_cast<const float4 *>(x + k + 4);
#pragma unroll
        for (int i = 0; i < NF; ++i) {
            const __nv_bfloat162 *pr = reinterpret_cast<const __nv_bfloat162 *>(&raw[i]);
            const float2 a = __bfloat1622float2(pr[0]), b = __bfloat1622float2(pr[1]), c = __bfloat1622float2(pr[2]), d = __bfloat1622float2(pr[3]);
            out[i] = fmaf(xa.x, a.x, fmaf(xa.y, a.y, fmaf(xa.z, b.x, fmaf(xa.w, b.y, out[i]))));
            out[i] = fmaf(xb.x, c.x, fmaf(xb.y, c.y, fmaf(xb.z, d.x, fmaf(xb.w, d.y, out[i]))));
        }
    }
#pragma unroll
    for (int i = 0; i < NF; ++i) out[i] = warp_sum(out[i]);
}

// act[(t top + s), f] = silu(Wg[e] h_t)[f] * (Wu[e] h_t)[f], e = ids[t, s].  A warp takes GU_PER_WARP features at once.
constexpr int GU_WARPS = 4, GU_PER_WARP = 4;
template <typename T>
__global__ void __launch_bounds__(GU_WARPS * 32) moe_gate_up_kernel(const T *__restrict__ h, int ldh, const int *__restrict__ ids, const T *__restrict__ wgu,
                                                                    T *__restrict__ act, int E, int F, int X, int top, int plain) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float hs[];       // the token's row
    const int row = blockIdx.x, t = row / top;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int k = threadIdx.x; k < E; k += blockDim.x) hs[k] = to_f32(act_load(h + (size_t)t * ldh + k));
    int e = act_load(ids + row);
    e = e < 0 ? 0 : (e >= X ? X - 1 : e);
    __syncthreads();
    const int f0 = (blockIdx.y * GU_WARPS + warp) * GU_PER_WARP;
    if (f0 >= F) return;
    if (plain) {
        // experts without a gate: wgu is [X, F, E] and act = relu(W_up h)^2
        const T *we = wgu + (size_t)e * F * E;
        if (sizeof(T) == 2 && (E % 8 == 0) && (reinterpret_cast<uintptr_t>(wgu) & 15) == 0) {
            const __nv_bfloat16 *rows[GU_PER_WARP];
#pragma unroll
            for (int i = 0; i < GU_PER_WARP; ++i) rows[i] = reinterpret_cast<const __nv_bfloat16 *>(we) + (size_t)min(f0 + i, F - 1) * E;
            float r[GU_PER_WARP];
            rows_dot_bf16<GU_PER_WARP>(rows, hs, E, lane, r);
            if (lane == 0)
#pragma unroll
                for (int i = 0; i < GU_PER_WARP; ++i)
                    if (f0 + i < F) {
                        const float a = fmaxf(r[i], 0.f);
                        act[(size_t)row * F + f0 + i] = from_f32<T>(a * a);
                    }
            return;
        }
        for (int f = f0; f < f0 + GU_PER_WARP && f < F; ++f) {
            const T *u_row = we + (size_t)f * E;
            float u = 0.f;
            for (int k = lane; k < E; k += 32) u = fmaf(hs[k], to_f32(u_row[k]), u);
            u = fmaxf(warp_sum(u), 0.f);
            if (lane == 0) act[(size_t)row * F + f] = from_f32<T>(u * u);
        }
        return;
    }
    // expert e's rows: gate of feature f at row 2 f, its up at row 2 f + 1
    const T *we = wgu + (size_t)e * 2 * F * E;
    if (sizeof(T) == 2 && (E % 8 == 0) && (reinterpret_cast<uintptr_t>(wgu) & 15) == 0) {
        const __nv_bfloat16 *rows[2 * GU_PER_WARP];
#pragma unroll
        for (int i = 0; i < GU_PER_WARP; ++i) {
            const int f = min(f0 + i, F - 1);
            rows[i] = reinterpret_cast<const __nv_bfloat16 *>(we) + (size_t)(2 * f) * E;
            rows[GU_PER_WARP + i] = rows[i] + E;
        }
        float r[2 * GU_PER_WARP];
        rows_dot_bf16<2 * GU_PER_WARP>(rows, hs, E, lane, r);
        if (lane == 0)
#pragma unroll
            for (int i = 0; i < GU_PER_WARP; ++i)
                if (f0 + i < F) act[(size_t)row * F + f0 + i] = from_f32<T>(r[i] / (1.0f + expf(-r[i])) * r[GU_PER_WARP + i]);
        return;
    }
    for (int f = f0; f < f0 + GU_PER_WARP && f < F; ++f) {
        const T *g_row = we + (size_t)(2 * f) * E, *u_row = g_row + E;
        float g = 0.f, u = 0.f;
        for (int k = lane; k < E; k += 32) {
            const float x = hs[k];
            g = fmaf(x, to_f32(g_row[k]), g);
            u = fmaf(x, to_f32(u_row[k]), u);
        }
        g = warp_sum(g);
        u = warp_sum(u);
        if (lane == 0) act[(size_t)row * F + f] = from_f32<T>(g / (1.0f + expf(-g)) * u);
    }
}

// out[t, j] = sum_s wts[t, s] (Wd[ids[t, s]] act[t top + s])[j], float32; the chosen experts in their order.  A warp takes
// DN_PER_WARP outputs at once.
constexpr int DN_WARPS = 4, DN_PER_WARP = 4;
template <typename T>
__global__ void __launch_bounds__(DN_WARPS * 32) moe_down_kernel(const T *__restrict__ act, const int *__restrict__ ids, const float *__restrict__ wts,
                                                                 const T *__restrict__ wd, float *__restrict__ out, int E, int F, int X, int top,
                                                                 const float *__restrict__ also, const float *__restrict__ also_w) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float as[];       // top rows of F
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int k = threadIdx.x; k < top * F; k += blockDim.x) as[k] = to_f32(act_load(act + (size_t)t * top * F + k));
    __syncthreads();
    const int j0 = (blockIdx.y * DN_WARPS + warp) * DN_PER_WARP;
    if (j0 >= E) return;
    const bool vec = sizeof(T) == 2 && (F % 8 == 0) && (reinterpret_cast<uintptr_t>(wd) & 15) == 0;
    float total[DN_PER_WARP];
#pragma unroll
    for (int i = 0; i < DN_PER_WARP; ++i) total[i] = 0.f;
    for (int s = 0; s < top; ++s) {
        int e = act_load(ids + (size_t)t * top + s);
        e = e < 0 ? 0 : (e >= X ? X - 1 : e);
        const float w = act_load(wts + (size_t)t * top + s);
        float r[DN_PER_WARP];
        if (vec) {
            const __nv_bfloat16 *rows[DN_PER_WARP];
#pragma unroll
            for (int i = 0; i < DN_PER_WARP; ++i) rows[i] = reinterpret_cast<const __nv_bfloat16 *>(wd) + ((size_t)e * E + min(j0 + i, E - 1)) * F;
            rows_dot_bf16<DN_PER_WARP>(rows, as + (size_t)s * F, F, lane, r);
        } else {
#pragma unroll
            for (int i = 0; i < DN_PER_WARP; ++i) {
                const T *d_row = wd + ((size_t)e * E + min(j0 + i, E - 1)) * F;
                float dot = 0.f;
                for (int k = lane; k < F; k += 32) dot = fmaf(as[(size_t)s * F + k], to_f32(d_row[k]), dot);
                r[i] = warp_sum(dot);
            }
        }
#pragma unroll
        for (int i = 0; i < DN_PER_WARP; ++i) total[i] = fmaf(w, r[i], total[i]);
    }
    // `also`: a term every token gets beside its chosen experts (a shared expert's output), times the token's own weight
    if (lane == 0)
#pragma unroll
        for (int i = 0; i < DN_PER_WARP; ++i)
            if (j0 + i < E) {
                float v = total[i];
                if (also) v = fmaf(act_load(also_w + t), act_load(also + (size_t)t * E + j0 + i), v);
                out[(size_t)t * E + j0 + i] = v;
            }
}

template <typename K>
static int need_smem(K kernel, size_t smem, const char *who) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LGML_FAIL("%s: cannot have %zu bytes of shared memory: %s", who, smem, cudaGetErrorString(e));
    }
    return 0;
}
}  // namespace

// h: [n, ldh] in the compute type; wr: float32 [X, E]; br: float32 [X] or null; ids int32 / wts float32 [n, top]
//   mode 0: the chosen by the largest logits + br, weights = softmax over the chosen logits
//   mode 1: scores = sigmoid(logits), the chosen by the largest score + br, weights = score / (sum of the chosen scores + 1e-20) * route_scale
//   wr holds n_extra more rows behind the experts': extra[n, n_extra] = sigmoid of their logits
LGML_API int lgml_moe_router_mode(const void *h, int dtype, int ldh, const float *wr, const float *br, int *ids, float *wts, int n_tokens, int E, int X,
                                  int top, int mode, float route_scale, int n_extra, float *extra, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && E > 0 && X > 0 && top > 0 && top <= X, "moe_router: bad sizes (%d experts, %d chosen)", X, top);
    LGML_REQUIRE(X <= 8192, "moe_router: at most 8192 experts");
    LGML_REQUIRE(mode == 0 || mode == 1, "moe_router: unknown mode %d", mode);
    LGML_REQUIRE(n_extra >= 0 && n_extra <= 64 && (n_extra == 0 || extra != nullptr), "moe_router: bad extra rows");
    if (n_tokens == 0) return 0;
    const size_t smem = sizeof(float) * (2 * (size_t)((X + n_extra + 3) & ~3) + (size_t)E);
    LGML_REQUIRE(smem <= 200 * 1024, "moe_router: %d experts and rows of %d do not fit shared memory", X, E);
    if (need_smem(moe_router_kernel<float>, smem, "moe_router") || need_smem(moe_router_kernel<__nv_bfloat16>, smem, "moe_router")) return -1;
    if (dtype == LGML_F32)
        lgml_launch(moe_router_kernel<float>, n_tokens, 128, smem, stream, (const float *)h, ldh, wr, br, ids, wts, E, X, top, mode, route_scale, n_extra, extra);
    else if (dtype == LGML_BF16)
        lgml_launch(moe_router_kernel<__nv_bfloat16>, n_tokens, 128, smem, stream, (const __nv_bfloat16 *)h, ldh, wr, br, ids, wts, E, X, top, mode,
                    route_scale, n_extra, extra);
    else
        LGML_FAIL("moe_router: unknown type %d", dtype);
    return lgml_launch_status("moe_router");
}

LGML_API int lgml_moe_router(const void *h, int dtype, int ldh, const float *wr, const float *br, int *ids, float *wts, int n_tokens, int E, int X,
                             int top, cudaStream_t stream) {
    return lgml_moe_router_mode(h, dtype, ldh, wr, br, ids, wts, n_tokens, E, X, top, 0, 1.0f, 0, nullptr, stream);
}

// The row form: act [n top, F] in the compute type (scratch of the caller), out float32 [n, E].
// plain = 1: experts without a gate (wgu is [X, F, E], act = relu(W_up h)^2).  also / also_w: float32 [n, E] and [n], out += also_w[t] also[t] (or null).
LGML_API int lgml_moe_experts_rows_form(const void *h, int dtype, int ldh, const int *ids, const float *wts, const void *wgu, const void *wd,
                                        void *act, float *out, int n_tokens, int E, int F, int X, int top, int plain, const float *also,
                                        const float *also_w, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && E > 0 && F > 0 && X > 0 && top > 0, "moe_experts_rows: bad sizes");
    if (n_tokens == 0) return 0;
    const size_t smem_gu = sizeof(float) * (size_t)E, smem_dn = sizeof(float) * (size_t)top * F;
    LGML_REQUIRE(smem_gu <= 200 * 1024 && smem_dn <= 200 * 1024, "moe_experts_rows: rows of %d or %d x %d floats do not fit shared memory", E, top, F);
    dim3 grid_gu(n_tokens * top, (F + GU_WARPS * GU_PER_WARP - 1) / (GU_WARPS * GU_PER_WARP));
    dim3 grid_dn(n_tokens, (E + DN_WARPS * DN_PER_WARP - 1) / (DN_WARPS * DN_PER_WARP));
    if (dtype == LGML_F32) {
        if (need_smem(moe_gate_up_kernel<float>, smem_gu, "moe_experts_rows") || need_smem(moe_down_kernel<float>, smem_dn, "moe_experts_rows")) return -1;
        lgml_launch(moe_gate_up_kernel<float>, grid_gu, GU_WARPS * 32, smem_gu, stream, (const float *)h, ldh, ids, (const float *)wgu, (float *)act, E, F, X,
                    top, plain);
        lgml_launch(moe_down_kernel<float>, grid_dn, DN_WARPS * 32, smem_dn, stream, (const float *)act, ids, wts, (const float *)wd, out, E, F, X, top,
                    also, also_w);
    } else if (dtype == LGML_BF16) {
        if (need_smem(moe_gate_up_kernel<__nv_bfloat16>, smem_gu, "moe_experts_rows") ||
            need_smem(moe_down_kernel<__nv_bfloat16>, smem_dn, "moe_experts_rows"))
            return -1;
        lgml_launch(moe_gate_up_kernel<__nv_bfloat16>, grid_gu, GU_WARPS * 32, smem_gu, stream, (const __nv_bfloat16 *)h, ldh, ids,
                    (const __nv_bfloat16 *)wgu, (__nv_bfloat16 *)act, E, F, X, top, plain);
        lgml_launch(moe_down_kernel<__nv_bfloat16>, grid_dn, DN_WARPS * 32, smem_dn, stream, (const __nv_bfloat16 *)act, ids, wts,
                    (const __nv_bfloat16 *)wd, out, E, F, X, top, also, also_w);
    } else {
        LGML_FAIL("moe_experts_rows: unknown type %d", dtype);
    }
    return lgml_launch_status("moe_experts_rows");
}

LGML_API int lgml_moe_experts_rows(const void *h, int dtype, int ldh, const int *ids, const float *wts, const void *wgu, const void *wd,
                                   void *act, float *out, int n_tokens, int E, int F, int X, int top, cudaStream_t stream) {
    return lgml_moe_experts_rows_form(h, dtype, ldh, ids, wts, wgu, wd, act, out, n_tokens, E, F, X, top, 0, nullptr, nullptr, stream);
}

// ---------------------------------------------------------------------------------------------
// The grouped form, bfloat16, for many tokens: the (token, chosen expert) rows are sorted by expert,
// cut into tiles of 128 rows of one expert, and every tile is a product on tensor cores (mma.sync
// m16n8k16, float32 accumulation) against that expert's matrices, which are then read once per tile
// and not once per row.
//   moe_group        counts the rows per expert, lists them expert by expert and writes the tiles
//                    (expert, first row of the list, rows); one block, no host in the loop, so the
//                    step stays a fixed sequence of launches whatever the router chose
//   moe_tile_product C[128 rows, 128 columns] of a tile: MODE 0 gathers the tokens' rows of h, takes 64
//                    gate and 64 up features at once and writes silu(gate) * up; MODE 1 reads the
//                    activations and writes the down product times the row's weight, float32
//   moe_sum          out[t] = the rows of token t added in the order of its chosen experts
// A row's result does not depend on where in a tile it lies, so the order in which rows were
// listed (atomics) does not show in the output.
// ---------------------------------------------------------------------------------------------
namespace {
constexpr int G_TM = 128, G_TN = 128, G_TK = 32, G_LD = G_TK + 8;

__global__ void __launch_bounds__(1024) moe_group_kernel(const int *__restrict__ ids, int n_rows, int X, int *__restrict__ rows,
                                                         int *__restrict__ tiles, int *__restrict__ n_tiles, int max_tiles) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ int sh[];         // counts[X], first[X], cursor[X], tile0[X]
    int *counts = sh, *first = sh + X, *cursor = sh + 2 * X, *tile0 = sh + 3 * X;
    for (int e = threadIdx.x; e < X; e += blockDim.x) counts[e] = 0, cursor[e] = 0;
    __syncthreads();
    for (int r = threadIdx.x; r < n_rows; r += blockDim.x) {
        int e = act_load(ids + r);
        e = e < 0 ? 0 : (e >= X ? X - 1 : e);
        atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tl = 0;
        for (int e = 0; e < X; ++e) {
            first[e] = at, tile0[e] = tl;
            at += counts[e];
            tl += (counts[e] + G_TM - 1) / G_TM;
        }
        *n_tiles = tl < max_tiles ? tl : max_tiles;
    }
    __syncthreads();
    for (int r = threadIdx.x; r < n_rows; r += blockDim.x) {
        int e = act_load(ids + r);
        e = e < 0 ? 0 : (e >= X ? X - 1 : e);
        rows[first[e] + atomicAdd(&cursor[e], 1)] = r;
    }
    for (int e = threadIdx.x; e < X; e += blockDim.x) {
        const int nt = (counts[e] + G_TM - 1) / G_TM;
        for (int i = 0; i < nt; ++i) {
            const int tl = tile0[e] + i;
            if (tl >= max_tiles) break;
            tiles[tl * 3] = e;
            tiles[tl * 3 + 1] = first[e] + i * G_TM;
            tiles[tl * 3 + 2] = min(G_TM, counts[e] - i * G_TM);
        }
    }
}

__device__ __forceinline__ uint32_t g_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void g_ldmatrix_x4(uint32_t (&r)[4], const void *p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(g_smem_u32(p)));
}
__device__ __forceinline__ void g_mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void g_cp16(void *dst, const void *src, bool valid) {
    const int bytes = valid ? 16 : 0;   // 0: zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(g_smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}

// MODE 0: a = h (rows gathered by token), b = 64 gate rows and the 64 up rows of the same features of w0[e] (pairs), from feature
//         64 blockIdx.y on (each of the two warp columns gets 32 gate and its 32 up features), out0 = act [n_rows, N] bfloat16.
//         K = E, N = F.
// MODE 1: a = act rows, b = 128 rows of w0[e] (down) from column 128 blockIdx.y on, out1 = y [n_rows, N] float32, times wts[row].
//         K = F, N = E.
// Eight warps, four down the rows and two across the columns: a warp owns 32 rows x 64 columns.  Three stages of cp.async.
constexpr int G_STAGES = 3;
constexpr int G_STAGE_ELEMS = (G_TM + G_TN) * G_LD;
template <int MODE>
__global__ void __launch_bounds__(256) moe_tile_product_kernel(const __nv_bfloat16 *__restrict__ a, int lda, const int *__restrict__ rows,
                                                               const int *__restrict__ tiles, const int *__restrict__ n_tiles,
                                                               const __nv_bfloat16 *__restrict__ w0, const float *__restrict__ wts, __nv_bfloat16 *__restrict__ out0,
                                                               float *__restrict__ out1, int K, int N, int top) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) uint8_t g_raw[];
    __nv_bfloat16 *stages = reinterpret_cast<__nv_bfloat16 *>(g_raw);
    int *row_of = reinterpret_cast<int *>(stages + G_STAGES * G_STAGE_ELEMS);
    const int tile = blockIdx.x;
    if (tile >= act_load(n_tiles)) return;
    const int e = act_load(tiles + tile * 3), r0 = act_load(tiles + tile * 3 + 1), n_r = act_load(tiles + tile * 3 + 2);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wm = warp & 3, wn = warp >> 2;
    const int mat = lane >> 3, mrow = lane & 7;
    if (threadIdx.x < G_TM) row_of[threadIdx.x] = threadIdx.x < n_r ? act_load(rows + r0 + threadIdx.x) : -1;
    __syncthreads();
    constexpr int HALF = G_TN / 2;
    const int c0 = MODE == 0 ? blockIdx.y * HALF : blockIdx.y * G_TN;     // first feature (MODE 0) or column (MODE 1)

    auto issue = [&](int kt, int buf) {
        const int k0 = kt * G_TK;
        __nv_bfloat16 *As = stages + (size_t)buf * G_STAGE_ELEMS, *Bs = As + G_TM * G_LD;
        for (int c = threadIdx.x; c < G_TM * (G_TK / 8); c += 256) {
            const int r = c / (G_TK / 8), col = (c - r * (G_TK / 8)) * 8;
            const int row = row_of[r];
            const bool ok = row >= 0 && k0 + col < K;
            const size_t src_row = MODE == 0 ? (size_t)(row >= 0 ? row / top : 0) : (size_t)(row >= 0 ? row : 0);
            g_cp16(As + r * G_LD + col, a + src_row * lda + (ok ? k0 + col : 0), ok);
        }
        for (int c = threadIdx.x; c < G_TN * (G_TK / 8); c += 256) {
            const int r = c / (G_TK / 8), col = (c - r * (G_TK / 8)) * 8;
            const __nv_bfloat16 *base;
            int n;
            if (MODE == 0) {
                const int half = r / 64, rr = r % 64;              // the warp column, and gate (rr < 32) or up
                n = c0 + half * 32 + (rr & 31);
                base = w0 + ((size_t)e * 2 * N + 2 * (n < N ? n : 0) + (rr < 32 ? 0 : 1)) * K;      // gate at row 2 n, up at 2 n + 1
            } else {
                n = c0 + r;
                base = w0 + ((size_t)e * N + (n < N ? n : 0)) * K;
            }
            const bool ok = n < N && k0 + col < K;
            g_cp16(Bs + r * G_LD + col, base + (ok ? k0 + col : 0), ok);
        }
    };
    float acc[2][8][4];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[m][i][0] = acc[m][i][1] = acc[m][i][2] = acc[m][i][3] = 0.f;
    const int n_kt = (K + G_TK - 1) / G_TK;
#pragma unroll
    for (int st = 0; st < G_STAGES - 1; ++st) {
        if (st < n_kt) issue(st, st);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int kt = 0; kt < n_kt; ++kt) {
        asm volatile("cp.async.wait_group %0;" ::"n"(G_STAGES - 2) : "memory");
        __syncthreads();            // stage kt has landed for everyone, and everyone is done with the buffer refilled next
        if (kt + G_STAGES - 1 < n_kt) issue(kt + G_STAGES - 1, (kt + G_STAGES - 1) % G_STAGES);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const __nv_bfloat16 *As = stages + (size_t)(kt % G_STAGES) * G_STAGE_ELEMS, *Bs = As + G_TM * G_LD;
#pragma unroll
        for (int ks = 0; ks < G_TK / 16; ++ks) {
            uint32_t af[2][4];
#pragma unroll
            for (int m = 0; m < 2; ++m)
                g_ldmatrix_x4(af[m], As + (wm * 32 + m * 16 + (mat & 1) * 8 + mrow) * G_LD + ks * 16 + (mat >> 1) * 8);
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t bq[4];
                g_ldmatrix_x4(bq, Bs + (wn * 64 + np * 16 + (mat >> 1) * 8 + mrow) * G_LD + ks * 16 + (mat & 1) * 8);
#pragma unroll
                for (int m = 0; m < 2; ++m) {
                    g_mma_bf16(acc[m][2 * np], af[m], bq[0], bq[1]);
                    g_mma_bf16(acc[m][2 * np + 1], af[m], bq[2], bq[3]);
                }
            }
        }
    }
    // rows lane / 4 and + 8 of each of the warp's two blocks of 16; columns 8 nt + (lane % 4) * 2 and + 1 of the warp's 64
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            const int r = wm * 32 + m * 16 + (lane >> 2) + rr * 8;
            const int row = row_of[r];
            if (row < 0) continue;
            if (MODE == 0) {
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int f = c0 + wn * 32 + nt * 8 + (lane & 3) * 2 + i;
                        if (f >= N) continue;
                        const float g = acc[m][nt][rr * 2 + i], u = acc[m][nt + 4][rr * 2 + i];
                        out0[(size_t)row * N + f] = __float2bfloat16_rn(g / (1.0f + expf(-g)) * u);
                    }
            } else {
                const float w = act_load(wts + row);
#pragma unroll
                for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int j = c0 + wn * 64 + nt * 8 + (lane & 3) * 2 + i;
                        if (j < N) out1[(size_t)row * N + j] = acc[m][nt][rr * 2 + i] * w;
                    }
            }
        }
}

__global__ void __launch_bounds__(256) moe_sum_kernel(const float *__restrict__ y, float *__restrict__ out, int n_tokens, int E, int top) {
    pdl_trigger();
    pdl_wait();
    const size_t total = (size_t)n_tokens * E;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / E, j = i - t * E;
        float s = 0.f;
        for (int k = 0; k < top; ++k) s += act_load(y + (t * top + k) * E + j);
        out[i] = s;
    }
}
}  // namespace

// h bfloat16 [n, ldh]; ids / wts [n, top]; the experts' matrices stacked, bfloat16; scratch of the caller: rows int32 [n top],
// tiles int32 [3 max_tiles + 1] (the last word: the number of tiles), act bfloat16 [n top, F], y float32 [n top, E];
// out float32 [n, E].  E and F multiples of 8, ldh too.
LGML_API int lgml_moe_experts_grouped(const void *h, int ldh, const int *ids, const float *wts, const void *wgu, const void *wd,
                                      int *rows, int *tiles, int max_tiles, void *act, float *y, float *out, int n_tokens, int E, int F, int X,
                                      int top, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && E > 0 && F > 0 && X > 0 && top > 0, "moe_experts_grouped: bad sizes");
    LGML_REQUIRE(E % 8 == 0 && F % 8 == 0 && ldh % 8 == 0, "moe_experts_grouped: widths %d, %d and the row stride %d must be multiples of 8", E, F, ldh);
    LGML_REQUIRE((((uintptr_t)h | (uintptr_t)wgu | (uintptr_t)wd | (uintptr_t)act) & 15) == 0, "moe_experts_grouped: operands must be 16-byte aligned");
    LGML_REQUIRE(X <= 8192, "moe_experts_grouped: at most 8192 experts");
    if (n_tokens == 0) return 0;
    const int n_rows = n_tokens * top;
    const int need = (n_rows + G_TM - 1) / G_TM + (X < n_rows ? X : n_rows);
    LGML_REQUIRE(max_tiles >= need, "moe_experts_grouped: room for %d tiles, %d may be needed", max_tiles, need);
    int *n_tiles = tiles + 3 * max_tiles;
    if (need_smem(moe_group_kernel, sizeof(int) * 4 * (size_t)X, "moe_experts_grouped")) return -1;
    lgml_launch(moe_group_kernel, 1, 1024, sizeof(int) * 4 * (size_t)X, stream, ids, n_rows, X, rows, tiles, n_tiles, max_tiles);
    dim3 g0(max_tiles, (F + G_TN / 2 - 1) / (G_TN / 2)), g1(max_tiles, (E + G_TN - 1) / G_TN);
    LGML_REQUIRE(g0.y <= 65535 && g1.y <= 65535, "moe_experts_grouped: too many columns");
    const size_t smem = (size_t)G_STAGES * G_STAGE_ELEMS * 2 + sizeof(int) * G_TM;
    if (need_smem(moe_tile_product_kernel<0>, smem, "moe_experts_grouped") || need_smem(moe_tile_product_kernel<1>, smem, "moe_experts_grouped")) return -1;
    lgml_launch(moe_tile_product_kernel<0>, g0, 256, smem, stream, (const __nv_bfloat16 *)h, ldh, (const int *)rows, (const int *)tiles,
                (const int *)n_tiles, (const __nv_bfloat16 *)wgu, (const float *)nullptr, (__nv_bfloat16 *)act, (float *)nullptr, E, F, top);
    lgml_launch(moe_tile_product_kernel<1>, g1, 256, smem, stream, (const __nv_bfloat16 *)act, F, (const int *)rows, (const int *)tiles,
                (const int *)n_tiles, (const __nv_bfloat16 *)wd, wts, (__nv_bfloat16 *)nullptr, y, F, E, top);
    const size_t total = (size_t)n_tokens * E;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    lgml_launch(moe_sum_kernel, blocks, 256, 0, stream, (const float *)y, out, n_tokens, E, top);
    return lgml_launch_status("moe_experts_grouped");
}

// ---------------------------------------------------------------------------------------------
// The pieces around a grouped product that another library computes (the tcgen05 product with a tile list):
//   moe_group_rows    the sorted rows and the tile list alone
//   moe_gather_rows   the tokens' rows of h copied into tiles of 128 rows, tile t holding the rows the list gives it, and
//                     where each (token, expert) row went
//   moe_weighted_sum  out[t] = sum_s wts[t, s] y[pos[t top + s]], the chosen experts in their order
// ---------------------------------------------------------------------------------------------
namespace {
__global__ void __launch_bounds__(128) moe_gather_rows_kernel(const __nv_bfloat16 *__restrict__ h, int ldh, const int *__restrict__ rows,
                                                              const int *__restrict__ tiles, int max_tiles, __nv_bfloat16 *__restrict__ a_perm,
                                                              int *__restrict__ pos, int E, int top) {
    pdl_trigger();
    pdl_wait();
    const int pr = blockIdx.x, tile = pr / G_TM, i = pr - tile * G_TM;
    if (tile >= act_load(tiles + 3 * max_tiles) || i >= act_load(tiles + 3 * tile + 2)) return;
    const int r = act_load(rows + act_load(tiles + 3 * tile + 1) + i);
    if (threadIdx.x == 0) pos[r] = pr;
    const uint4 *src = reinterpret_cast<const uint4 *>(h + (size_t)(r / top) * ldh);
    uint4 *dst = reinterpret_cast<uint4 *>(a_perm + (size_t)pr * E);
    for (int c = threadIdx.x; c < E / 8; c += blockDim.x) dst[c] = act_load(src + c);
}

__global__ void __launch_bounds__(256) moe_weighted_sum_kernel(const float *__restrict__ y, const int *__restrict__ pos, const float *__restrict__ wts,
                                                               float *__restrict__ out, int n_tokens, int E, int top,
                                                               const float *__restrict__ also, const float *__restrict__ also_w) {
    pdl_trigger();
    pdl_wait();
    if (E % 4 == 0 && ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(also)) & 15) == 0) {
        const int quads = E / 4;
        const size_t total = (size_t)n_tokens * quads;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
            const size_t t = i / quads, j = (i - t * quads) * 4;
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int k = 0; k < top; ++k) {
                const float w = act_load(wts + t * top + k);
                const float4 v = act_load(reinterpret_cast<const float4 *>(y + (size_t)act_load(pos + t * top + k) * E + j));
                s.x = fmaf(w, v.x, s.x), s.y = fmaf(w, v.y, s.y), s.z = fmaf(w, v.z, s.z), s.w = fmaf(w, v.w, s.w);
            }
            if (also) {
                const float w = act_load(also_w + t);
                const float4 v = act_load(reinterpret_cast<const float4 *>(also + t * E + j));
                s.x = fmaf(w, v.x, s.x), s.y = fmaf(w, v.y, s.y), s.z = fmaf(w, v.z, s.z), s.w = fmaf(w, v.w, s.w);
            }
            *reinterpret_cast<float4 *>(out + t * E + j) = s;
        }
        return;
    }
    const size_t total = (size_t)n_tokens * E;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / E, j = i - t * E;
        float s = 0.f;
        for (int k = 0; k < top; ++k) s = fmaf(act_load(wts + t * top + k), act_load(y + (size_t)act_load(pos + t * top + k) * E + j), s);
        if (also) s = fmaf(act_load(also_w + t), act_load(also + i), s);
        out[i] = s;
    }
}
}  // namespace

// rows int32 [n top]; tiles int32 [3 max_tiles + 1] (the last word: the number of tiles)
LGML_API int lgml_moe_group_rows(const int *ids, int *rows, int *tiles, int max_tiles, int n_tokens, int X, int top, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && X > 0 && X <= 8192 && top > 0, "moe_group_rows: bad sizes");
    const int n_rows = n_tokens * top;
    const int need = (n_rows + G_TM - 1) / G_TM + (X < n_rows ? X : n_rows);
    LGML_REQUIRE(max_tiles >= need, "moe_group_rows: room for %d tiles, %d may be needed", max_tiles, need);
    if (n_tokens == 0) return 0;
    if (need_smem(moe_group_kernel, sizeof(int) * 4 * (size_t)X, "moe_group_rows")) return -1;
    lgml_launch(moe_group_kernel, 1, 1024, sizeof(int) * 4 * (size_t)X, stream, ids, n_rows, X, rows, tiles, tiles + 3 * max_tiles, max_tiles);
    return lgml_launch_status("moe_group_rows");
}

// a_perm bfloat16 [max_tiles 128, E]; pos int32 [n top]
LGML_API int lgml_moe_gather_rows(const void *h, int ldh, const int *rows, const int *tiles, int max_tiles, void *a_perm, int *pos, int E, int top,
                                  cudaStream_t stream) {
    LGML_REQUIRE(max_tiles > 0 && E > 0 && E % 8 == 0 && ldh % 8 == 0 && top > 0, "moe_gather_rows: bad sizes");
    LGML_REQUIRE((((uintptr_t)h | (uintptr_t)a_perm) & 15) == 0, "moe_gather_rows: operands must be 16-byte aligned");
    lgml_launch(moe_gather_rows_kernel, max_tiles * G_TM, 128, 0, stream, (const __nv_bfloat16 *)h, ldh, rows, tiles, max_tiles, (__nv_bfloat16 *)a_perm, pos,
                E, top);
    return lgml_launch_status("moe_gather_rows");
}

LGML_API int lgml_moe_weighted_sum_also(const float *y, const int *pos, const float *wts, float *out, int n_tokens, int E, int top, const float *also,
                                        const float *also_w, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && E > 0 && top > 0, "moe_weighted_sum: bad sizes");
    if (n_tokens == 0) return 0;
    const size_t total = (size_t)n_tokens * E;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    lgml_launch(moe_weighted_sum_kernel, blocks, 256, 0, stream, y, pos, wts, out, n_tokens, E, top, also, also_w);
    return lgml_launch_status("moe_weighted_sum");
}

LGML_API int lgml_moe_weighted_sum(const float *y, const int *pos, const float *wts, float *out, int n_tokens, int E, int top, cudaStream_t stream) {
    return lgml_moe_weighted_sum_also(y, pos, wts, out, n_tokens, E, top, nullptr, nullptr, stream);
}
