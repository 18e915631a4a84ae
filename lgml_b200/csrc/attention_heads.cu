// What some attention mixers do per head around the attention itself.
//
//   diff_combine     differential attention: a head has two attention maps over the same values;
//                    o = a1 - lambda a2, then o / rms(o) * out_scale, per head
//   latent_prepare   latent attention: the down-projection's first R columns, RMS-normed, are the
//                    latent c; its last Dr columns are a rotated key part shared by all heads;
//                    both go into one cell of the cache [c | k_rot].  The queries' rotated part is
//                    rotated and placed behind the R columns that head_linear fills
//   head_linear      a product per head (FMA units; tensor cores from 32 tokens on): out[t, h, :] = W[h] x[t, h, :], for the up-projections of
//                    latent attention taken to the query side (q W_uk) and to the output side
//                    (W_uv o), so that attention itself runs on the cached latent
//
// Norms, angles and the combination are float32 in both compute types.
#include <math.h>

#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_attention_heads)

namespace {
constexpr int MAX_DV = 512;

// in: [n, 2 H Dv], the maps in the order (key head g, map m, query head r of the group): map m of
// head h = g per + r lies at head slot (2 g + m) per + r.  out: [n, H Dv].
template <typename TI, typename TO>
__global__ void __launch_bounds__(128) diff_combine_kernel(const TI *__restrict__ in, int ldi, TO *__restrict__ out, int ldo, int H, int G,
                                                           int Dv, float lambda, float eps, float out_scale) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int per = H / G;
    for (int h = warp; h < H; h += n_warps) {
        const int g = h / per, r = h - g * per;
        const TI *a1 = in + (size_t)t * ldi + (size_t)((2 * g) * per + r) * Dv;
        const TI *a2 = in + (size_t)t * ldi + (size_t)((2 * g + 1) * per + r) * Dv;
        float o[MAX_DV / 32];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < MAX_DV / 32; ++i) {
            const int d = lane + 32 * i;
            o[i] = 0.f;
            if (d < Dv) {
                o[i] = to_f32(act_load(a1 + d)) - lambda * to_f32(act_load(a2 + d));
                ss = fmaf(o[i], o[i], ss);
            }
        }
        ss = warp_sum(ss);
        const float inv = out_scale / sqrtf(ss / (float)Dv + eps);
#pragma unroll
        for (int i = 0; i < MAX_DV / 32; ++i) {
            const int d = lane + 32 * i;
            if (d < Dv) out[(size_t)t * ldo + (size_t)h * Dv + d] = from_f32<TO>(o[i] * inv);
        }
    }
}

// One block per token.  qp: float32 [n, H (D + Dr)] (per head: D plain, Dr rotated); dkv: float32
// [n, R + Dr].  Rotation: the first n_rot of the Dr entries, pairs (2i, 2i + 1), angle
// pos * (freq[i] + freq_lo[i]); the rest pass unchanged.
template <typename T>
__global__ void __launch_bounds__(128) latent_prepare_kernel(
    const float *__restrict__ qp, int ldqp, const float *__restrict__ dkv, int lddkv, const float *__restrict__ norm_w, float eps,
    const float *__restrict__ freq, const float *__restrict__ freq_lo, int n_rot, const int *__restrict__ positions,
    const int *__restrict__ seq_of_token, const int *__restrict__ block_table, int max_blocks, T *__restrict__ k_pages, int n_pages,
    int page_size, T *__restrict__ q_plain, int ldqplain, T *__restrict__ q_full, int ldqfull, int H, int D, int Dr, int R, int write_kv,
    float rot_mag, int *__restrict__ status) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float cs[];       // cos, then sin, of the n_rot / 2 angles
    __shared__ float red[32];
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = n_rot / 2;
    float *sn = cs + half;
    // rot_mag: a factor on every cosine and sine (frequency scalings that lengthen the rotated vectors); 1 changes no bit
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sv, cv;
        rope_sincos(pos, freq[i], freq_lo ? freq_lo[i] : 0.f, &sv, &cv);
        sn[i] = sv * rot_mag, cs[i] = cv * rot_mag;
    }
    const float *drow = dkv + (size_t)t * lddkv;
    float ss = 0.f;
    if (write_kv)
        for (int k = threadIdx.x; k < R; k += blockDim.x) {
            const float v = act_load(drow + k);
            ss = fmaf(v, v, ss);
        }
    ss = block_sum(ss, red);            // (also the barrier behind the angles)
    if (write_kv) {
        const int seq = seq_of_token[t];
        const int blk = pos / page_size;
        int page = -1;
        if (pos >= 0 && blk < max_blocks) page = block_table[(size_t)seq * max_blocks + blk];
        if (page < 0 || page >= n_pages) {      // the host reserves pages first; never write outside the pool
            if (threadIdx.x == 0) atomicExch(status, 2);
        } else {
            const float inv = 1.0f / sqrtf(ss / (float)R + eps);
            T *cell = k_pages + ((size_t)page * page_size + (size_t)(pos % page_size)) * (R + Dr);
            for (int k = threadIdx.x; k < R; k += blockDim.x) cell[k] = from_f32<T>(act_load(drow + k) * inv * norm_w[k]);
            for (int i = threadIdx.x; i < half; i += blockDim.x) {
                const float u = act_load(drow + R + 2 * i), v = act_load(drow + R + 2 * i + 1);
                cell[R + 2 * i] = from_f32<T>(u * cs[i] - v * sn[i]);
                cell[R + 2 * i + 1] = from_f32<T>(v * cs[i] + u * sn[i]);
            }
            for (int d = n_rot + threadIdx.x; d < Dr; d += blockDim.x) cell[R + d] = from_f32<T>(act_load(drow + R + d));
        }
    }
    const float *qrow = qp + (size_t)t * ldqp;
    for (int e = threadIdx.x; e < H * D; e += blockDim.x) {
        const int h = e / D, d = e - h * D;
        q_plain[(size_t)t * ldqplain + e] = from_f32<T>(act_load(qrow + (size_t)h * (D + Dr) + d));
    }
    for (int e = threadIdx.x; e < H * half; e += blockDim.x) {
        const int h = e / half, i = e - h * half;
        const float *src = qrow + (size_t)h * (D + Dr) + D;
        const float u = act_load(src + 2 * i), v = act_load(src + 2 * i + 1);
        T *dst = q_full + (size_t)t * ldqfull + (size_t)h * (R + Dr) + R;
        dst[2 * i] = from_f32<T>(u * cs[i] - v * sn[i]);
        dst[2 * i + 1] = from_f32<T>(v * cs[i] + u * sn[i]);
    }
    const int rest = Dr - n_rot;
    for (int e = threadIdx.x; e < H * rest; e += blockDim.x) {
        const int h = e / rest, d = n_rot + (e - h * rest);
        q_full[(size_t)t * ldqfull + (size_t)h * (R + Dr) + R + d] = from_f32<T>(act_load(qrow + (size_t)h * (D + Dr) + D + d));
    }
}

// an output gate: the product times sigmoid(gate[t, h oh + o]) (float32 logits of a projection of the mixer's input)
__device__ __forceinline__ float gate_sigmoid(float g) { return 1.0f / (1.0f + expf(-g)); }

// out[t, h oh + o] = sum_k x[t, h xh + k] w[h][o][k]; float32 sums, k in order, so a row's result
// does not depend on what else is in the batch.  A block: 32 tokens x 64 outputs of one head.
constexpr int HL_TM = 32, HL_TN = 64, HL_TK = 32;
template <typename T>
__global__ void __launch_bounds__(256) head_linear_kernel(const T *__restrict__ x, int ldx, int xh, const T *__restrict__ w, T *__restrict__ out,
                                                          int ldo, int oh, int n, int O, int K, const float *__restrict__ gate, int ldg) {
    pdl_trigger();
    pdl_wait();
    __shared__ float xs[HL_TM][HL_TK + 1];
    __shared__ float ws[HL_TN][HL_TK + 1];
    const int h = blockIdx.z, t0 = blockIdx.x * HL_TM, o0 = blockIdx.y * HL_TN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const T *wh = w + (size_t)h * O * K;
    float acc[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += HL_TK) {
        for (int e = threadIdx.x; e < HL_TM * HL_TK; e += blockDim.x) {
            const int r = e / HL_TK, c = e - r * HL_TK;
            xs[r][c] = (t0 + r < n && k0 + c < K) ? to_f32(act_load(x + (size_t)(t0 + r) * ldx + (size_t)h * xh + k0 + c)) : 0.f;
        }
        for (int e = threadIdx.x; e < HL_TN * HL_TK; e += blockDim.x) {
            const int r = e / HL_TK, c = e - r * HL_TK;
            ws[r][c] = (o0 + r < O && k0 + c < K) ? to_f32(wh[(size_t)(o0 + r) * K + k0 + c]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < HL_TK; ++kk) {
            float a[2], b[4];
#pragma unroll
            for (int i = 0; i < 2; ++i) a[i] = xs[ty + 16 * i][kk];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[tx + 16 * j][kk];
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int t = t0 + ty + 16 * i, o = o0 + tx + 16 * j;
            if (t < n && o < O) {
                float v = acc[i][j];
                if (gate) v *= gate_sigmoid(act_load(gate + (size_t)t * ldg + (size_t)h * oh + o));
                out[(size_t)t * ldo + (size_t)h * oh + o] = from_f32<T>(v);
            }
        }
}

// The same product on tensor cores (mma.sync m16n8k16, float32 accumulation) for many tokens, bfloat16: a block of four
// warps takes 64 tokens x 64 outputs of one head, K in steps of 64 through shared memory (16-byte cp.async, zeros past
// the edges); a warp owns 16 tokens.  A row's sums do not depend on which tile it lies in.
constexpr int HM_T = 64, HM_K = 64, HM_LD = HM_K + 8;
__device__ __forceinline__ uint32_t hm_smem(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__global__ void __launch_bounds__(128) head_linear_mma_kernel(const __nv_bfloat16 *__restrict__ x, int ldx, int xh, const __nv_bfloat16 *__restrict__ w,
                                                              __nv_bfloat16 *__restrict__ out, int ldo, int oh, int n, int O, int K,
                                                              const float *__restrict__ gate, int ldg) {
    pdl_trigger();
    pdl_wait();
    __shared__ __align__(16) __nv_bfloat16 As[HM_T * HM_LD];
    __shared__ __align__(16) __nv_bfloat16 Bs[HM_T * HM_LD];
    const int h = blockIdx.z, t0 = blockIdx.x * HM_T, o0 = blockIdx.y * HM_T;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int mat = lane >> 3, mrow = lane & 7;
    const __nv_bfloat16 *wh = w + (size_t)h * O * K;
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    for (int k0 = 0; k0 < K; k0 += HM_K) {
        for (int c = threadIdx.x; c < HM_T * (HM_K / 8); c += 128) {
            const int r = c / (HM_K / 8), col = (c - r * (HM_K / 8)) * 8;
            const bool oka = t0 + r < n && k0 + col < K, okb = o0 + r < O && k0 + col < K;
            const __nv_bfloat16 *sa = x + (size_t)(oka ? t0 + r : 0) * ldx + (size_t)h * xh + (oka ? k0 + col : 0);
            const __nv_bfloat16 *sb = wh + (size_t)(okb ? o0 + r : 0) * K + (okb ? k0 + col : 0);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(hm_smem(As + r * HM_LD + col)), "l"(sa), "r"(oka ? 16 : 0) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(hm_smem(Bs + r * HM_LD + col)), "l"(sb), "r"(okb ? 16 : 0) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < HM_K / 16; ++ks) {
            uint32_t a[4];
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                         : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
                         : "r"(hm_smem(As + (warp * 16 + (mat & 1) * 8 + mrow) * HM_LD + ks * 16 + (mat >> 1) * 8)));
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b[4];
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                             : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3])
                             : "r"(hm_smem(Bs + (np * 16 + (mat >> 1) * 8 + mrow) * HM_LD + ks * 16 + (mat & 1) * 8)));
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                             : "+f"(acc[2 * np][0]), "+f"(acc[2 * np][1]), "+f"(acc[2 * np][2]), "+f"(acc[2 * np][3])
                             : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                             : "+f"(acc[2 * np + 1][0]), "+f"(acc[2 * np + 1][1]), "+f"(acc[2 * np + 1][2]), "+f"(acc[2 * np + 1][3])
                             : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[2]), "r"(b[3]));
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int t = t0 + warp * 16 + (lane >> 2) + rr * 8;
        if (t >= n) continue;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int o = o0 + nt * 8 + (lane & 3) * 2 + i;
                if (o < O) {
                    float v = acc[nt][rr * 2 + i];
                    if (gate) v *= gate_sigmoid(act_load(gate + (size_t)t * ldg + (size_t)h * oh + o));
                    out[(size_t)t * ldo + (size_t)h * oh + o] = __float2bfloat16_rn(v);
                }
            }
    }
}
}  // namespace

LGML_API int lgml_diff_combine(const void *in, int in_dtype, int ldi, void *out, int out_dtype, int ldo, int n_tokens, int H, int G, int Dv,
                               float lambda, float eps, float out_scale, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && H > 0 && G > 0 && Dv > 0, "diff_combine: bad sizes");
    LGML_REQUIRE(H % G == 0, "diff_combine: %d heads are no multiple of %d key heads", H, G);
    LGML_REQUIRE(Dv <= MAX_DV, "diff_combine: value size %d must be at most %d", Dv, MAX_DV);
    LGML_REQUIRE(ldi >= 2 * H * Dv && ldo >= H * Dv, "diff_combine: row strides below the rows");
    if (n_tokens == 0) return 0;
#define LGML_DC(TI, TO) lgml_launch(diff_combine_kernel<TI, TO>, n_tokens, 128, 0, stream, (const TI *)in, ldi, (TO *)out, ldo, H, G, Dv, lambda, eps, out_scale)
    if (in_dtype == LGML_F32 && out_dtype == LGML_F32) LGML_DC(float, float);
    else if (in_dtype == LGML_F32 && out_dtype == LGML_BF16) LGML_DC(float, __nv_bfloat16);
    else if (in_dtype == LGML_BF16 && out_dtype == LGML_BF16) LGML_DC(__nv_bfloat16, __nv_bfloat16);
    else LGML_FAIL("diff_combine: types %d -> %d are not built", in_dtype, out_dtype);
#undef LGML_DC
    return lgml_launch_status("diff_combine");
}

LGML_API int lgml_latent_prepare(const float *qp, int ldqp, const float *dkv, int lddkv, const float *norm_w, float eps, const float *freq,
                                 const float *freq_lo, int n_rot, const int *positions, const int *seq_of_token, const int *block_table,
                                 int max_blocks, void *k_pages, int dtype, int n_pages, int page_size, void *q_plain, int ldqplain, void *q_full,
                                 int ldqfull, int n_tokens, int H, int D, int Dr, int R, int write_kv, float rot_mag, int *status, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && H > 0 && D > 0 && Dr >= 0 && R > 0 && page_size > 0 && max_blocks > 0, "latent_prepare: bad sizes");
    LGML_REQUIRE(n_rot >= 0 && n_rot <= Dr && n_rot % 2 == 0, "latent_prepare: %d rotated entries of %d", n_rot, Dr);
    LGML_REQUIRE(ldqp >= H * (D + Dr) && lddkv >= R + Dr && ldqplain >= H * D && ldqfull >= H * (R + Dr), "latent_prepare: row strides below the rows");
    if (n_tokens == 0) return 0;
    const size_t smem = sizeof(float) * (size_t)(n_rot > 0 ? n_rot : 1);
    LGML_REQUIRE(smem <= 48 * 1024, "latent_prepare: %d rotated entries are too many", n_rot);
    if (dtype == LGML_F32)
        lgml_launch(latent_prepare_kernel<float>, n_tokens, 128, smem, stream, qp, ldqp, dkv, lddkv, norm_w, eps, freq, freq_lo, n_rot, positions,
                    seq_of_token, block_table, max_blocks, (float *)k_pages, n_pages, page_size, (float *)q_plain, ldqplain, (float *)q_full, ldqfull,
                    H, D, Dr, R, write_kv, rot_mag, status);
    else if (dtype == LGML_BF16)
        lgml_launch(latent_prepare_kernel<__nv_bfloat16>, n_tokens, 128, smem, stream, qp, ldqp, dkv, lddkv, norm_w, eps, freq, freq_lo, n_rot,
                    positions, seq_of_token, block_table, max_blocks, (__nv_bfloat16 *)k_pages, n_pages, page_size, (__nv_bfloat16 *)q_plain,
                    ldqplain, (__nv_bfloat16 *)q_full, ldqfull, H, D, Dr, R, write_kv, rot_mag, status);
    else
        LGML_FAIL("latent_prepare: unknown type %d", dtype);
    return lgml_launch_status("latent_prepare");
}

// x: [n, ldx] with head h at column h xh; w: [H, O, K] contiguous; out: [n, ldo] with head h at column h oh.
LGML_API int lgml_head_linear(const void *x, int ldx, int xh, const void *w, void *out, int ldo, int oh, int dtype, int n_tokens, int H, int O,
                              int K, const float *gate, int ldg, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && H > 0 && O > 0 && K > 0, "head_linear: bad sizes");
    LGML_REQUIRE(H <= 65535 && (O + HL_TN - 1) / HL_TN <= 65535, "head_linear: too many heads or outputs");
    if (n_tokens == 0) return 0;
    if (dtype == LGML_BF16 && n_tokens >= 32 && K % 8 == 0 && ldx % 8 == 0 && xh % 8 == 0 && (((uintptr_t)x | (uintptr_t)w) & 15) == 0) {
        dim3 gm((n_tokens + HM_T - 1) / HM_T, (O + HM_T - 1) / HM_T, H);
        lgml_launch(head_linear_mma_kernel, gm, 128, 0, stream, (const __nv_bfloat16 *)x, ldx, xh, (const __nv_bfloat16 *)w, (__nv_bfloat16 *)out, ldo, oh,
                    n_tokens, O, K, gate, ldg);
        return lgml_launch_status("head_linear");
    }
    dim3 grid((n_tokens + HL_TM - 1) / HL_TM, (O + HL_TN - 1) / HL_TN, H);
    if (dtype == LGML_F32)
        lgml_launch(head_linear_kernel<float>, grid, 256, 0, stream, (const float *)x, ldx, xh, (const float *)w, (float *)out, ldo, oh, n_tokens, O, K, gate, ldg);
    else if (dtype == LGML_BF16)
        lgml_launch(head_linear_kernel<__nv_bfloat16>, grid, 256, 0, stream, (const __nv_bfloat16 *)x, ldx, xh, (const __nv_bfloat16 *)w,
                    (__nv_bfloat16 *)out, ldo, oh, n_tokens, O, K, gate, ldg);
    else
        LGML_FAIL("head_linear: unknown type %d", dtype);
    return lgml_launch_status("head_linear");
}
