// Attention with a sink, a distance bias and a window over the paged cache, for mixers whose
// keys and values have head sizes of their own (D for q and k, Dv for v).
//
//   score(i, j) = (q_i . k_j) * scale - slope_h * (i - j)        for 0 <= i - j < window (0: all j <= i)
//   weight(i, j) = exp(score(i, j)) / (exp(sink_h) + sum_j' exp(score(i, j')))
//   out_i = sum_j weight(i, j) v_j      [* sigmoid(gate_i) element by element, when a gate is given]
//
// The sink is one more term of the denominator: it has no key and no value.  Scores, the running
// maximum, the sums and the gate are float32 in both compute types.
//
// Two kernels.  sink_qkv_store takes the fused projection's float32 output (q | k | v [| more]),
// multiplies q by its position's temperature 1 + coef * ln(floor((p + 1) / every) + 1), mixes v
// with the values another layer kept for the same token (v <- (1 - lambda) v + lambda v_first), and
// stores k and the mixed v in their cells and q in its own buffer.  sink_attention is the general
// form: one block per (token, head); a (token, head)'s result depends only on that token's
// position and its request's cells, read in a fixed order, so it is the same however the tokens
// were cut into steps and whatever else is in the batch.
#include <math.h>

#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_attention_sink)

namespace {

// A cap on the scaled scores: cap tanh(s / cap) (cap 0: none), applied before the distance bias.
// capped_score2 gives the result in the base-2 domain (times log2 e).
__device__ __forceinline__ float capped_score(float dot, float scale, float cap) {
    const float s = dot * scale;
    return cap > 0.f ? cap * tanhf(s / cap) : s;
}
__device__ __forceinline__ float capped_score2(float dot, float scale, float cap) {
    return cap * 1.4426950408889634f * tanhf(dot * scale / cap);
}
constexpr int ITEMS = 256;
constexpr int WARPS = 4;
constexpr int MAX_D = 256;        // the split decode forms (a lane holds 8 value columns)
constexpr int GEN_MAX_D = 512;    // the general form

// v_mode: 0 store v as it is; 1 also keep it in v_keep (float32 [tokens, Hkv Dv]); 2 mix with v_keep first
template <typename T>
__global__ void __launch_bounds__(ITEMS) sink_qkv_store_kernel(
    const float *__restrict__ proj, int ldp, T *__restrict__ q_out, int ldq, const int *__restrict__ positions,
    const int *__restrict__ seq_of_token, const int *__restrict__ block_table, int max_blocks, T *__restrict__ k_pages,
    T *__restrict__ v_pages, int n_pages, int page_size, int H, int Hkv, int Hv, int D, int Dv, float temp_coef, int temp_every,
    int v_mode, float *__restrict__ v_keep, const float *__restrict__ v_lambda, int write_kv, int *__restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int nq = H * D, nk = Hkv * D, nv = Hv * Dv;
    const int e = blockIdx.y * ITEMS + threadIdx.x;
    if (e >= nq + (write_kv ? nk + nv : 0)) return;
    const int pos = positions[t];
    float val = act_load(proj + (size_t)t * ldp + e);
    if (e < nq) {
        if (temp_coef != 0.f) val *= 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f);
        q_out[(size_t)t * ldq + e] = from_f32<T>(val);
        return;
    }
    const int seq = seq_of_token[t];
    const int blk = pos / page_size;
    int page = -1;
    if (pos >= 0 && blk < max_blocks) page = block_table[(size_t)seq * max_blocks + blk];
    if (page < 0 || page >= n_pages) {   // the host reserves pages first; never write outside the pool
        if (e == nq) atomicExch(status, 2);
        return;
    }
    if (e < nq + nk) {
        const int c = e - nq, g = c / D, d = c - g * D;
        k_pages[(((size_t)page * Hkv + g) * page_size + (size_t)(pos % page_size)) * D + d] = from_f32<T>(val);
        return;
    }
    const int c = e - nq - nk, g = c / Dv, d = c - g * Dv;
    if (v_mode == 1) {
        v_keep[(size_t)t * nv + c] = val;
    } else if (v_mode == 2) {
        const float lam = v_lambda[0];
        val = (1.0f - lam) * val + lam * act_load(v_keep + (size_t)t * nv + c);
    }
    v_pages[(((size_t)page * Hv + g) * page_size + (size_t)(pos % page_size)) * Dv + d] = from_f32<T>(val);
}

template <typename T, typename TO>
__global__ void __launch_bounds__(WARPS * 32) sink_attention_kernel(
    const T *__restrict__ q, int ldq, const int *__restrict__ positions, const int *__restrict__ seq_of_token,
    const int *__restrict__ block_table, int max_blocks, const T *__restrict__ k_pages, const T *__restrict__ v_pages,
    int n_pages, int page_size, const float *__restrict__ slopes, const float *__restrict__ sinks,
    const float *__restrict__ gate, int ldg, TO *__restrict__ out, int ldo, int H, int Hkv, int Hv, int D, int Dv, int ldv, float scale, float softcap,
    int window, int keep_first, int *__restrict__ status) {
    pdl_trigger();
    pdl_wait();
    __shared__ float qs[GEN_MAX_D];
    __shared__ float acc_w[WARPS][GEN_MAX_D];
    __shared__ float m_w[WARPS], l_w[WARPS];
    const int t = blockIdx.x, h = blockIdx.y;
    const int g = h / (H / Hkv);
    const int gv = g / (Hkv / Hv);          // several key heads may share one value head
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = positions[t];
    const int seq = seq_of_token[t];
    const int *table = block_table + (size_t)seq * max_blocks;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int n_first = keep_first < lo ? keep_first : lo;     // kept first tokens that the window does not hold anyway
    const int n_keys = n_first + (pos - lo + 1);
    const float slope = slopes ? slopes[h] : 0.f;

    for (int d = threadIdx.x; d < D; d += blockDim.x) qs[d] = to_f32(act_load(q + (size_t)t * ldq + (size_t)h * D + d));
    __syncthreads();

    float m = -INFINITY, l = 0.f;
    float acc[GEN_MAX_D / 32];
#pragma unroll
    for (int i = 0; i < GEN_MAX_D / 32; ++i) acc[i] = 0.f;

    // the visible keys in order: the kept first tokens, then the window; warp w takes every WARPS-th
    for (int i = warp; i < n_keys; i += WARPS) {
        const int j = i < n_first ? i : lo + (i - n_first);
        const int blk = j / page_size;
        const int page = blk < max_blocks ? table[blk] : -1;
        if (page < 0 || page >= n_pages) {  // a cell the table does not hold: flag it, skip the key
            if (lane == 0) atomicExch(status, 3);
            continue;
        }
        const size_t cell = ((size_t)page * Hkv + g) * page_size + (size_t)(j % page_size);
        const size_t vcell = ((size_t)page * Hv + gv) * page_size + (size_t)(j % page_size);
        float dot = 0.f;
        for (int d = lane; d < D; d += 32) dot = fmaf(qs[d], to_f32(act_load(k_pages + cell * D + d)), dot);
        const float s = capped_score(warp_sum(dot), scale, softcap) - slope * (float)(pos - j);
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);  // exp(-inf) = 0 on the first key
        const float p = expf(s - m_new);
        l = l * corr + p;
#pragma unroll
        for (int i2 = 0; i2 < GEN_MAX_D / 32; ++i2) {
            const int d = lane + 32 * i2;
            if (d < Dv) acc[i2] = acc[i2] * corr + p * to_f32(act_load(v_pages + vcell * ldv + d));
        }
        m = m_new;
    }
    if (lane == 0) {
        m_w[warp] = m;
        l_w[warp] = l;
    }
#pragma unroll
    for (int i = 0; i < GEN_MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < Dv) acc_w[warp][d] = acc[i];
    }
    __syncthreads();
    const float sink = sinks ? sinks[h] : -INFINITY;
    float mm = sink;
    for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, m_w[w]);
    float lsum = sinks ? expf(sink - mm) : 0.f;
    float f[WARPS];
    for (int w = 0; w < WARPS; ++w) {
        f[w] = (m_w[w] == -INFINITY) ? 0.f : expf(m_w[w] - mm);
        lsum += l_w[w] * f[w];
    }
    for (int d = threadIdx.x; d < Dv; d += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < WARPS; ++w) o += acc_w[w][d] * f[w];
        o = lsum > 0.f ? o / lsum : 0.f;
        if (gate) o *= 1.0f / (1.0f + expf(-act_load(gate + (size_t)t * ldg + (size_t)h * Dv + d)));
        out[(size_t)t * ldo + (size_t)h * Dv + d] = from_f32<TO>(o);
    }
}

// ---------------------------------------------------------------------------------------------
// Prompts and portions, bfloat16, on tensor cores (mma.sync m16n8k16, float32 accumulation).
// A CTA of four warps takes a tile of up to 64 consecutive tokens of one request and one head; a
// warp owns 16 query rows.  The keys are walked a page (64 keys) at a time, only the pages the
// tile's window reaches: S = Q K^T with Q as the A operand (fragments held in registers for the
// whole walk) and the page's keys as B; scale, distance bias and the causal/window mask on the
// accumulators; a running maximum and sum per row; P, rounded to bfloat16, goes straight from
// the accumulators' layout into the A operand of O += P V.  At the end the sink joins the
// denominator, and the gate multiplies the output.  KS = key size / 16 and NV = value size / 8
// (both rounded up; the padding is zeros in shared memory).
// ---------------------------------------------------------------------------------------------
constexpr int TILE_Q = 64;
constexpr int PAGE = 64;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void *p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void *p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the hardware's approximation (two units in the last place; -inf gives 0): the weights
// it makes are rounded to bfloat16 for the second product
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// a result as bfloat16, or as float32 for a caller that combines heads afterwards
__device__ __forceinline__ void store_out(void *out, int out_f32, size_t idx, float v) {
    if (out_f32) reinterpret_cast<float *>(out)[idx] = v;
    else reinterpret_cast<__nv_bfloat16 *>(out)[idx] = __float2bfloat16_rn(v);
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

// rows x width elements from global (row r at src + r * ld... given by row_ptr(r), null: zeros) into
// shared rows of `lds` elements, zero-padded to `padded` columns; 16-byte loads when `vec`
template <typename RowPtr>
__device__ __forceinline__ void load_rows(__nv_bfloat16 *dst, int lds, int rows, int width, int padded, bool vec, RowPtr row_ptr) {
    const int chunks = padded / 8;
    for (int c = threadIdx.x; c < rows * chunks; c += blockDim.x) {
        const int r = c / chunks, col = (c - r * chunks) * 8;
        const __nv_bfloat16 *src = row_ptr(r);
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (src != nullptr) {
            if (vec && col + 8 <= width) {
                val = act_load(reinterpret_cast<const uint4 *>(src + col));
            } else {
                __nv_bfloat16 *e = reinterpret_cast<__nv_bfloat16 *>(&val);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (col + j < width) e[j] = act_load(src + col + j);
            }
        }
        *reinterpret_cast<uint4 *>(dst + (size_t)r * lds + col) = val;
    }
}

template <int KS, int NV>
__global__ void __launch_bounds__(128, 3) sink_attention_mma_kernel(
    const __nv_bfloat16 *__restrict__ q, int ldq, const int *__restrict__ positions, const int *__restrict__ tiles,
    const int *__restrict__ block_table, int max_blocks, const __nv_bfloat16 *__restrict__ k_pages,
    const __nv_bfloat16 *__restrict__ v_pages, int n_pages, const float *__restrict__ slopes, const float *__restrict__ sinks,
    const float *__restrict__ gate, int ldg, void *__restrict__ out, int out_f32, int ldo, int H, int Hkv, int Hv, int D, int Dv, int ldv,
    float scale, float softcap, int window, int keep_first, int *__restrict__ status) {
    pdl_trigger();
    pdl_wait();
    constexpr int DP = KS * 16, DVP = NV * 8;
    constexpr int LDK = DP + 8, LDV = DVP + 8;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    // two buffers of keys, then two of values; the queries lie in the second buffer of keys until
    // their fragments are in registers (that buffer is first written for the second page)
    __nv_bfloat16 *Ks = reinterpret_cast<__nv_bfloat16 *>(smem_raw);
    __nv_bfloat16 *Qs = Ks + PAGE * LDK;
    __nv_bfloat16 *Vs = Ks + 2 * PAGE * LDK;
    const int tile = blockIdx.x, h = blockIdx.y;
    const int g = h / (H / Hkv);
    const int gv = g / (Hkv / Hv);
    const int seq = tiles[tile * 4], row0 = tiles[tile * 4 + 1], n_tok = tiles[tile * 4 + 2];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int mat = lane >> 3, mrow = lane & 7;
    const int p0 = positions[row0];                       // the tile's tokens stand at p0, p0 + 1, ...
    const int p_last = p0 + n_tok - 1;
    const int lo_key = (window > 0 && p0 - window + 1 > 0) ? p0 - window + 1 : 0;
    const int *table = block_table + (size_t)seq * max_blocks;
    const bool vec_k = (D % 8 == 0) && (ldq % 8 == 0) && ((reinterpret_cast<uintptr_t>(q) & 15) == 0);
    const float LOG2E = 1.4426950408889634f;
    const float slope2 = (slopes ? slopes[h] : 0.f) * LOG2E, scale2 = scale * LOG2E;

    load_rows(Qs, LDK, TILE_Q, D, DP, vec_k, [&](int r) { return r < n_tok ? q + (size_t)(row0 + r) * ldq + (size_t)h * D : nullptr; });
    __syncthreads();
    uint32_t qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) ldmatrix_x4(qf[ks], Qs + (size_t)(warp * 16 + (mat & 1) * 8 + mrow) * LDK + ks * 16 + (mat >> 1) * 8);

    // this thread's two rows of the warp's 16: r0 = lane / 4 and r0 + 8
    const int qr[2] = {warp * 16 + (lane >> 2), warp * 16 + (lane >> 2) + 8};
    const int qpos[2] = {p0 + qr[0], p0 + qr[1]};
    const bool qok[2] = {qr[0] < n_tok, qr[1] < n_tok};
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float oacc[NV][4];
#pragma unroll
    for (int i = 0; i < NV; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;

    // With rows of whole 16-byte pieces the pages come by cp.async into two buffers in turn: the
    // copy of the next page runs under the products of this one.  Else one buffer, plain loads.
    const bool pipelined = (D % 8 == 0) && (Dv % 8 == 0) && (ldv % 8 == 0) && ((reinterpret_cast<uintptr_t>(v_pages) & 15) == 0);
    const int pg_first = lo_key / PAGE, pg_last = p_last / PAGE;
    // the pages walked: those of the kept first tokens that lie before the window's, then the window's
    const int n_kp = window > 0 ? min((keep_first + PAGE - 1) / PAGE, pg_first) : 0;
    const int n_iter = n_kp + pg_last - pg_first + 1;
    auto page_at = [&](int it) { return it < n_kp ? it : pg_first + (it - n_kp); };
    auto issue = [&](int pg, int buf) {
        const int page = pg < max_blocks ? table[pg] : -1;
        const bool have = page >= 0 && page < n_pages;
        if (!have && threadIdx.x == 0) atomicExch(status, 3);
        const size_t cell0 = ((size_t)(have ? page : 0) * Hkv + g) * PAGE;
        const size_t vcell0 = ((size_t)(have ? page : 0) * Hv + gv) * PAGE;
        __nv_bfloat16 *Kb = Ks + (size_t)buf * PAGE * LDK, *Vb = Vs + (size_t)buf * PAGE * LDV;
        for (int c = threadIdx.x; c < PAGE * (DP / 8); c += blockDim.x) {
            const int r = c / (DP / 8), col = (c - r * (DP / 8)) * 8;
            const int bytes = (have && col < D) ? 16 : 0;       // 0: zeros
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(Kb + (size_t)r * LDK + col)),
                         "l"(k_pages + (cell0 + r) * D + (col < D ? col : 0)), "r"(bytes) : "memory");
        }
        for (int c = threadIdx.x; c < PAGE * (DVP / 8); c += blockDim.x) {
            const int r = c / (DVP / 8), col = (c - r * (DVP / 8)) * 8;
            const int bytes = (have && col < Dv) ? 16 : 0;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(Vb + (size_t)r * LDV + col)),
                         "l"(v_pages + (vcell0 + r) * ldv + (col < Dv ? col : 0)), "r"(bytes) : "memory");
        }
    };
    if (pipelined) {
        issue(page_at(0), 0);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int it = 0; it < n_iter; ++it) {
        const int pg = page_at(it);
        const int buf = pipelined ? (it & 1) : 0;
        const __nv_bfloat16 *Kb = Ks + (size_t)buf * PAGE * LDK, *Vb = Vs + (size_t)buf * PAGE * LDV;
        __syncthreads();            // everyone is done with the page before: its buffer is free
        if (pipelined) {
            if (it + 1 < n_iter) issue(page_at(it + 1), buf ^ 1);
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            const int page = pg < max_blocks ? table[pg] : -1;
            const bool have = page >= 0 && page < n_pages;
            if (!have && threadIdx.x == 0) atomicExch(status, 3);
            const size_t cell0 = ((size_t)(have ? page : 0) * Hkv + g) * PAGE;
            const size_t vcell0 = ((size_t)(have ? page : 0) * Hv + gv) * PAGE;
            load_rows(Ks, LDK, PAGE, D, DP, false, [&](int r) { return have ? k_pages + (cell0 + r) * D : nullptr; });
            load_rows(Vs, LDV, PAGE, Dv, DVP, false, [&](int r) { return have ? v_pages + (vcell0 + r) * ldv : nullptr; });
        }
        __syncthreads();
        // the warp's rows see keys up to their own positions: skip a page that lies wholly outside
        const int w_first = p0 + warp * 16, w_last = min(w_first + 15, p_last);
        const int key0 = pg * PAGE;
        if (warp * 16 >= n_tok || key0 > w_last || (window > 0 && key0 + PAGE - 1 < w_first - window + 1 && key0 >= keep_first)) continue;

        float sacc[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {       // two key tiles of 8 per ldmatrix
                uint32_t b[4];
                ldmatrix_x4(b, Kb + (size_t)(np * 16 + (mat >> 1) * 8 + mrow) * LDK + ks * 16 + (mat & 1) * 8);
                mma_bf16(sacc[2 * np], qf[ks], b[0], b[1]);
                mma_bf16(sacc[2 * np + 1], qf[ks], b[2], b[3]);
            }
        }
        // scale, distance bias, mask; scores in the base-2 domain.  Most pages lie wholly inside the
        // window and before the warp's first row: there every key counts, and the bias of element
        // (row, key) is a row term plus a key term, one multiply-add and one add a score.
        float mx[2] = {-INFINITY, -INFINITY};
        const bool interior = key0 + PAGE - 1 <= w_first && (window == 0 || w_last - key0 < window);
        if (interior) {
            const float rowt[2] = {-slope2 * (float)(qpos[0] - key0), -slope2 * (float)(qpos[1] - key0)};
            const float colb = slope2 * (float)((lane & 3) * 2);
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float bias2 = rowt[i >> 1] + fmaf(slope2, (float)(nt * 8 + (i & 1)), colb);
                    const float sv = softcap > 0.f ? capped_score2(sacc[nt][i], scale, softcap) + bias2 : fmaf(sacc[nt][i], scale2, bias2);
                    sacc[nt][i] = sv;
                    mx[i >> 1] = fmaxf(mx[i >> 1], sv);
                }
        } else {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int rr = i >> 1;
                    const int j = key0 + nt * 8 + (lane & 3) * 2 + (i & 1);
                    const int dist = qpos[rr] - j;
                    const bool ok = qok[rr] && dist >= 0 && (window == 0 || dist < window || j < keep_first);
                    const float sv = ok ? (softcap > 0.f ? capped_score2(sacc[nt][i], scale, softcap) : sacc[nt][i] * scale2) - slope2 * (float)dist : -INFINITY;
                    sacc[nt][i] = sv;
                    mx[rr] = fmaxf(mx[rr], sv);
                }
        }
        float corr[2], m_use[2];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
            mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
            const float m_new = fmaxf(m_run[rr], mx[rr]);
            corr[rr] = (m_new == -INFINITY) ? 1.f : fast_exp2(m_run[rr] - m_new);
            m_run[rr] = m_new;
            m_use[rr] = (m_new == -INFINITY) ? 0.f : m_new;       // a row that has seen no key yet: every weight is exp2(-inf) = 0
            l_run[rr] *= corr[rr];
        }
        uint32_t pf[4][4];           // P as A fragments: key step kk covers key tiles 2 kk and 2 kk + 1
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            float pv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) pv[i] = fast_exp2(sacc[nt][i] - m_use[i >> 1]);
            l_run[0] += pv[0] + pv[1];
            l_run[1] += pv[2] + pv[3];
            pf[nt >> 1][(nt & 1) * 2] = pack_bf16(pv[0], pv[1]);
            pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(pv[2], pv[3]);
        }
#pragma unroll
        for (int nv = 0; nv < NV; ++nv) {
            oacc[nv][0] *= corr[0];
            oacc[nv][1] *= corr[0];
            oacc[nv][2] *= corr[1];
            oacc[nv][3] *= corr[1];
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int np = 0; np < NV / 2; ++np) {   // two value tiles of 8 per ldmatrix
                uint32_t b[4];
                ldmatrix_x4_trans(b, Vb + (size_t)(kk * 16 + (mat & 1) * 8 + mrow) * LDV + np * 16 + (mat >> 1) * 8);
                mma_bf16(oacc[2 * np], pf[kk], b[0], b[1]);
                mma_bf16(oacc[2 * np + 1], pf[kk], b[2], b[3]);
            }
        }
    }
    // the sink joins the denominator; the quad's partial sums are added up
    const float sink2 = sinks ? sinks[h] * LOG2E : -INFINITY;
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 1);
        l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 2);
        const float m_all = fmaxf(m_run[rr], sink2);
        const float f = (m_run[rr] == -INFINITY) ? 0.f : exp2f(m_run[rr] - m_all);
        const float den = l_run[rr] * f + (sinks ? exp2f(sink2 - m_all) : 0.f);
        const float inv = den > 0.f ? f / den : 0.f;
        if (!qok[rr]) continue;
        const size_t t = (size_t)(row0 + qr[rr]);
#pragma unroll
        for (int nv = 0; nv < NV; ++nv)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int d = nv * 8 + (lane & 3) * 2 + e;
                if (d >= Dv) continue;
                float o = oacc[nv][rr * 2 + e] * inv;
                if (gate) o *= 1.0f / (1.0f + __expf(-act_load(gate + t * ldg + (size_t)h * Dv + d)));
                store_out(out, out_f32, t * ldo + (size_t)h * Dv + d, o);
            }
    }
}

template <int KS, int NV>
int launch_mma(dim3 grid, cudaStream_t stream, const __nv_bfloat16 *q, int ldq, const int *positions, const int *tiles, const int *block_table,
               int max_blocks, const __nv_bfloat16 *k_pages, const __nv_bfloat16 *v_pages, int n_pages, const float *slopes, const float *sinks,
               const float *gate, int ldg, void *out, int out_f32, int ldo, int H, int Hkv, int Hv, int D, int Dv, int ldv, float scale, float softcap, int window,
               int keep_first, int *status) {
    const size_t smem = ((size_t)2 * PAGE * (KS * 16 + 8) + (size_t)2 * PAGE * (NV * 8 + 8)) * 2;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(sink_attention_mma_kernel<KS, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LGML_FAIL("sink_attention_mma: cannot have %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    lgml_launch(sink_attention_mma_kernel<KS, NV>, grid, 128, smem, stream, q, ldq, positions, tiles, block_table, max_blocks, k_pages, v_pages,
                n_pages, slopes, sinks, gate, ldg, out, out_f32, ldo, H, Hkv, Hv, D, Dv, ldv, scale, softcap, window, keep_first, status);
    return lgml_launch_status("sink_attention_mma");
}

// ---------------------------------------------------------------------------------------------
// Decoding and short portions, bfloat16: every query token on its own, its keys cut into
// `n_splits` ranges of 32-key blocks.  A CTA takes (token, KV head [x chunk of up to GH of its
// query heads], range): the query heads that share a KV head are scored together, so each key and
// value is read once for all of them.  Within a warp the two halves of the work are laid out
// differently, so that neither needs a reduction across lanes per key: for q . k every lane owns
// one key of a block of 32 and reads its whole row; for the weighted sum of v every lane owns a few
// value columns and walks the block's keys, with the weights passed through shared memory.  All
// loads of a block are independent of each other and go out together.  A range leaves an
// unnormalised partial result (maximum, sum, weighted values); sink_decode_combine merges the
// ranges in order, lets the sink join the denominator and applies the gate.
// ---------------------------------------------------------------------------------------------
constexpr int DEC_WARPS = 4;
constexpr int DEC_COLS = 8;        // value columns per lane: two chunks of 4 (VEC), or 8 strided ones
constexpr int DEC_MAX_SPLITS = 64;

template <int GH, bool VEC>
__global__ void __launch_bounds__(DEC_WARPS * 32) sink_decode_kernel(
    const __nv_bfloat16 *__restrict__ q, int ldq, const int *__restrict__ positions, const int *__restrict__ seq_of_token,
    const int *__restrict__ block_table, int max_blocks, const __nv_bfloat16 *__restrict__ k_pages,
    const __nv_bfloat16 *__restrict__ v_pages, int n_pages, const float *__restrict__ slopes, const float *__restrict__ sinks,
    const float *__restrict__ gate, int ldg, void *__restrict__ out, int out_f32, int ldo, float *__restrict__ part_o,
    float2 *__restrict__ part_ml, int n_splits, int n_chunks, int H, int Hkv, int Hv, int D, int Dv, int ldv, float scale, float softcap, int window,
    int keep_first, int v_stage, int *__restrict__ status) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float dsm[];
    float *qs = dsm;                                   // [GH][D]
    float *ps = qs + GH * D;                           // [WARPS][GH][32]
    float *mw = ps + DEC_WARPS * GH * 32;              // [WARPS][GH] maxima, then [WARPS][GH] sums
    float *lw = mw + DEC_WARPS * GH;
    float *ow = lw + DEC_WARPS * GH;                   // [WARPS][GH][Dv]
    // [WARPS][32][Dv] bfloat16 when v_stage: a block's values, copied while its scores are computed
    __nv_bfloat16 *vstage = reinterpret_cast<__nv_bfloat16 *>(ow + DEC_WARPS * GH * Dv) + (size_t)(threadIdx.x >> 5) * 32 * Dv;
    const int t = blockIdx.x;
    const int g = blockIdx.y / n_chunks, chunk = blockIdx.y - g * n_chunks;
    const int split = blockIdx.z;
    const int group = H / Hkv;
    const int h0 = g * group + chunk * GH;
    const int g_count = min(GH, group - chunk * GH);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = positions[t];
    const int *table = block_table + (size_t)seq_of_token[t] * max_blocks;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const float LOG2E = 1.4426950408889634f;
    const float scale2 = scale * LOG2E;

    for (int i = threadIdx.x; i < GH * D; i += blockDim.x) {
        const int hh = i / D, d = i - hh * D;
        qs[i] = hh < g_count ? __bfloat162float(act_load(q + (size_t)t * ldq + (size_t)(h0 + hh) * D + d)) : 0.f;
    }
    __syncthreads();
    float slope2[GH];
#pragma unroll
    for (int hh = 0; hh < GH; ++hh) slope2[hh] = (slopes && hh < g_count) ? slopes[h0 + hh] * LOG2E : 0.f;

    // blocks of 32 keys: those of the kept first tokens that lie before the window's, then the window's
    const int b_lo = lo / 32, b_hi = pos / 32;
    const int n_kb = window > 0 ? min((keep_first + 31) / 32, b_lo) : 0;
    const int n_blocks = n_kb + b_hi - b_lo + 1;
    const int per = (n_blocks + n_splits - 1) / n_splits;
    const int b0 = split * per, b1 = min(b0 + per, n_blocks);
    const int gv = g / (Hkv / Hv);

    float m_run[GH], l_run[GH], acc[GH][DEC_COLS];
#pragma unroll
    for (int hh = 0; hh < GH; ++hh) {
        m_run[hh] = -INFINITY;
        l_run[hh] = 0.f;
#pragma unroll
        for (int c = 0; c < DEC_COLS; ++c) acc[hh][c] = 0.f;
    }
    float *pw = ps + warp * GH * 32;
    for (int bi = b0 + warp; bi < b1; bi += DEC_WARPS) {
        const int b = bi < n_kb ? bi : b_lo + (bi - n_kb);
        const int pg = b >> 1;
        const int page = pg < max_blocks ? table[pg] : -1;
        if (page < 0 || page >= n_pages) {
            if (lane == 0) atomicExch(status, 3);
            continue;
        }
        const size_t cell0 = ((size_t)page * Hkv + g) * PAGE + (size_t)(b & 1) * 32;     // the block's first cell
        const size_t vcell0 = ((size_t)page * Hv + gv) * PAGE + (size_t)(b & 1) * 32;
        const int j = b * 32 + lane;
        const bool ok = (j >= lo || j < keep_first) && j <= pos;
        // the values read: from the first visible key to the last (a key between kept tokens and window weighs 0)
        const int k_first = b * 32 < keep_first ? 0 : max(lo - b * 32, 0);
        const int k_last = b * 32 + 31 < lo ? min(keep_first - b * 32, 32) - 1 : min(pos - b * 32, 31);
        const __nv_bfloat16 *vbase = v_pages + vcell0 * ldv;
        if (v_stage) {
            // the block's visible values on their way into shared memory (through L2) while the scores are computed
            const int chunks = Dv / 8;
            for (int c = lane; c < (k_last - k_first + 1) * chunks; c += 32) {
                const int kk = k_first + c / chunks, d = (c % chunks) * 8;
                const uint32_t dst = (uint32_t)__cvta_generic_to_shared(vstage + (size_t)kk * Dv + d);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(vbase + (size_t)kk * ldv + d) : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        float sc[GH];
#pragma unroll
        for (int hh = 0; hh < GH; ++hh) sc[hh] = 0.f;
        if (ok) {
            const __nv_bfloat16 *krow = k_pages + (cell0 + lane) * D;
            if (VEC) {
                // sixteen 16-byte loads (128 elements of the key's row) go out before the first is used
                for (int c0 = 0; c0 < D; c0 += 128) {
                    uint4 raw[16];
#pragma unroll
                    for (int u = 0; u < 16; ++u)
                        if (c0 + u * 8 < D) raw[u] = act_load(reinterpret_cast<const uint4 *>(krow + c0 + u * 8));
#pragma unroll
                    for (int u = 0; u < 16; ++u) {
                        const int c = c0 + u * 8;
                        if (c >= D) break;
                        const __nv_bfloat162 *pr = reinterpret_cast<const __nv_bfloat162 *>(&raw[u]);
                        float kf[8];
#pragma unroll
                        for (int v2 = 0; v2 < 4; ++v2) {
                            const float2 f = __bfloat1622float2(pr[v2]);
                            kf[2 * v2] = f.x;
                            kf[2 * v2 + 1] = f.y;
                        }
#pragma unroll
                        for (int hh = 0; hh < GH; ++hh) {
                            const float4 qa = *reinterpret_cast<const float4 *>(qs + hh * D + c), qb = *reinterpret_cast<const float4 *>(qs + hh * D + c + 4);
                            sc[hh] = fmaf(qa.x, kf[0], fmaf(qa.y, kf[1], fmaf(qa.z, kf[2], fmaf(qa.w, kf[3], sc[hh]))));
                            sc[hh] = fmaf(qb.x, kf[4], fmaf(qb.y, kf[5], fmaf(qb.z, kf[6], fmaf(qb.w, kf[7], sc[hh]))));
                        }
                    }
                }
            } else {
                for (int d = 0; d < D; ++d) {
                    const float kf = __bfloat162float(act_load(krow + d));
#pragma unroll
                    for (int hh = 0; hh < GH; ++hh) sc[hh] = fmaf(qs[hh * D + d], kf, sc[hh]);
                }
            }
        }
        float corr[GH];
#pragma unroll
        for (int hh = 0; hh < GH; ++hh) {
            const float sv = ok ? (softcap > 0.f ? capped_score2(sc[hh], scale, softcap) : sc[hh] * scale2) - slope2[hh] * (float)(pos - j) : -INFINITY;
            const float m_new = fmaxf(m_run[hh], warp_max(sv));
            corr[hh] = (m_new == -INFINITY) ? 1.f : exp2f(m_run[hh] - m_new);
            const float p = (m_new == -INFINITY) ? 0.f : exp2f(sv - m_new);
            m_run[hh] = m_new;
            l_run[hh] = l_run[hh] * corr[hh] + p;          // this lane's keys; the lanes are added up at the end
            pw[hh * 32 + lane] = p;
        }
        __syncwarp();
#pragma unroll
        for (int hh = 0; hh < GH; ++hh)
#pragma unroll
            for (int c = 0; c < DEC_COLS; ++c) acc[hh][c] *= corr[hh];
        if (v_stage) {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncwarp();
            for (int kk = k_first; kk <= k_last; ++kk) {
                float vf[DEC_COLS];
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int d = (lane + 32 * i) * 4;
                    float2 raw = make_float2(0.f, 0.f);
                    if (d < Dv) raw = *reinterpret_cast<const float2 *>(vstage + (size_t)kk * Dv + d);
                    const __nv_bfloat162 *pr = reinterpret_cast<const __nv_bfloat162 *>(&raw);
                    const float2 f0 = __bfloat1622float2(pr[0]), f1 = __bfloat1622float2(pr[1]);
                    vf[4 * i] = f0.x, vf[4 * i + 1] = f0.y, vf[4 * i + 2] = f1.x, vf[4 * i + 3] = f1.y;
                }
#pragma unroll
                for (int hh = 0; hh < GH; ++hh) {
                    const float p = pw[hh * 32 + kk];
#pragma unroll
                    for (int c = 0; c < DEC_COLS; ++c) acc[hh][c] = fmaf(p, vf[c], acc[hh][c]);
                }
            }
        } else if (VEC) {
            // eight keys at a time: their loads go out together
            for (int kb = k_first; kb <= k_last; kb += 8) {
                float2 raw[8][2];
#pragma unroll
                for (int u = 0; u < 8; ++u)
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int d = (lane + 32 * i) * 4;
                        raw[u][i] = (kb + u <= k_last && d < Dv) ? act_load(reinterpret_cast<const float2 *>(vbase + (size_t)(kb + u) * ldv + d))
                                                                 : make_float2(0.f, 0.f);
                    }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    if (kb + u > k_last) break;
                    float vf[DEC_COLS];
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const __nv_bfloat162 *pr = reinterpret_cast<const __nv_bfloat162 *>(&raw[u][i]);
                        const float2 f0 = __bfloat1622float2(pr[0]), f1 = __bfloat1622float2(pr[1]);
                        vf[4 * i] = f0.x, vf[4 * i + 1] = f0.y, vf[4 * i + 2] = f1.x, vf[4 * i + 3] = f1.y;
                    }
#pragma unroll
                    for (int hh = 0; hh < GH; ++hh) {
                        const float p = pw[hh * 32 + kb + u];
#pragma unroll
                        for (int c = 0; c < DEC_COLS; ++c) acc[hh][c] = fmaf(p, vf[c], acc[hh][c]);
                    }
                }
            }
        } else {
            for (int kk = k_first; kk <= k_last; ++kk) {
                float vf[DEC_COLS];
                const __nv_bfloat16 *vrow = vbase + (size_t)kk * ldv;
#pragma unroll
                for (int c = 0; c < DEC_COLS; ++c) {
                    const int d = lane + 32 * c;
                    vf[c] = d < Dv ? __bfloat162float(act_load(vrow + d)) : 0.f;
                }
#pragma unroll
                for (int hh = 0; hh < GH; ++hh) {
                    const float p = pw[hh * 32 + kk];
#pragma unroll
                    for (int c = 0; c < DEC_COLS; ++c) acc[hh][c] = fmaf(p, vf[c], acc[hh][c]);
                }
            }
        }
        __syncwarp();
    }
    // the four warps' partial results, merged in warp order
#pragma unroll
    for (int hh = 0; hh < GH; ++hh) {
        const float l = warp_sum(l_run[hh]);
        if (lane == 0) {
            mw[warp * GH + hh] = m_run[hh];
            lw[warp * GH + hh] = l;
        }
#pragma unroll
        for (int c = 0; c < DEC_COLS; ++c) {
            const int d = VEC ? (lane + 32 * (c >> 2)) * 4 + (c & 3) : lane + 32 * c;
            if (d < Dv) ow[((size_t)warp * GH + hh) * Dv + d] = acc[hh][c];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < g_count * Dv; i += blockDim.x) {
        const int hh = i / Dv, d = i - hh * Dv;
        float m = -INFINITY;
        for (int w = 0; w < DEC_WARPS; ++w) m = fmaxf(m, mw[w * GH + hh]);
        float o = 0.f, l = 0.f;
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float f = (mw[w * GH + hh] == -INFINITY) ? 0.f : exp2f(mw[w * GH + hh] - m);
            o += ow[((size_t)w * GH + hh) * Dv + d] * f;
            l += lw[w * GH + hh] * f;
        }
        const int h = h0 + hh;
        if (n_splits == 1) {
            const float sink2 = sinks ? sinks[h] * LOG2E : -INFINITY;
            const float m_all = fmaxf(m, sink2);
            const float f = (m == -INFINITY) ? 0.f : exp2f(m - m_all);
            const float den = l * f + (sinks ? exp2f(sink2 - m_all) : 0.f);
            float r = den > 0.f ? o * f / den : 0.f;
            if (gate) r *= 1.0f / (1.0f + __expf(-act_load(gate + (size_t)t * ldg + (size_t)h * Dv + d)));
            store_out(out, out_f32, (size_t)t * ldo + (size_t)h * Dv + d, r);
        } else {
            part_o[(((size_t)t * H + h) * n_splits + split) * Dv + d] = o;
            if (d == 0) part_ml[((size_t)t * H + h) * n_splits + split] = make_float2(m, l);
        }
    }
}

__global__ void __launch_bounds__(128) sink_decode_combine_kernel(const float *__restrict__ part_o, const float2 *__restrict__ part_ml,
                                                                  const float *__restrict__ sinks, const float *__restrict__ gate, int ldg,
                                                                  void *__restrict__ out, int out_f32, int ldo, int n_splits, int H, int Dv) {
    pdl_trigger();
    pdl_wait();
    __shared__ float f_s[DEC_MAX_SPLITS];
    __shared__ float inv_s;
    const int t = blockIdx.x, h = blockIdx.y;
    const float2 *ml = part_ml + ((size_t)t * H + h) * n_splits;
    if (threadIdx.x == 0) {
        float m = -INFINITY;
        for (int i = 0; i < n_splits; ++i) m = fmaxf(m, act_load(ml + i).x);
        const float sink2 = sinks ? sinks[h] * 1.4426950408889634f : -INFINITY;
        const float m_all = fmaxf(m, sink2);
        float den = sinks ? exp2f(sink2 - m_all) : 0.f;
        for (int i = 0; i < n_splits; ++i) {
            const float2 v = act_load(ml + i);
            const float f = (v.x == -INFINITY) ? 0.f : exp2f(v.x - m_all);
            f_s[i] = f;
            den += v.y * f;
        }
        inv_s = den > 0.f ? 1.0f / den : 0.f;
    }
    __syncthreads();
    const float *po = part_o + ((size_t)t * H + h) * n_splits * Dv;
    for (int d = threadIdx.x; d < Dv; d += blockDim.x) {
        float o = 0.f;
        for (int i = 0; i < n_splits; ++i) o += act_load(po + (size_t)i * Dv + d) * f_s[i];
        o *= inv_s;
        if (gate) o *= 1.0f / (1.0f + __expf(-act_load(gate + (size_t)t * ldg + (size_t)h * Dv + d)));
        store_out(out, out_f32, (size_t)t * ldo + (size_t)h * Dv + d, o);
    }
}

// ---------------------------------------------------------------------------------------------
// The same split, on tensor cores, for head sizes that are multiples of 32 up to 128.  With one
// query per head the products are turned round: the keys are the M side of the tile and the (up
// to 8) heads of a KV head the N side:
//     S^T[64 keys, 8 heads] = K[64, D] . Q^T[D, 8]          O^T[Dv, 8 heads] += V^T[Dv, 64] . P^T[64, 8]
// Each of the four warps is a pipeline of its own over 16 keys of every page (cp.async, STAGES
// deep), with a running maximum, sum and output of its own; the four are merged once at the end.
// The distance bias and the window act on the score fragments; the sink and the gate come in
// where the result is normalised (here, or in sink_decode_combine when the keys were cut).
// ---------------------------------------------------------------------------------------------
constexpr int NH = 8;
__device__ __forceinline__ void cp_async_16z(void *dst, const void *src, bool valid) {
    const int bytes = valid ? 16 : 0;   // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}

template <int KS, int VS, int STAGES>
__global__ void __launch_bounds__(DEC_WARPS * 32) sink_decode_mma_kernel(
    const __nv_bfloat16 *__restrict__ q, int ldq, const int *__restrict__ positions, const int *__restrict__ seq_of_token,
    const int *__restrict__ block_table, int max_blocks, const __nv_bfloat16 *__restrict__ k_pages,
    const __nv_bfloat16 *__restrict__ v_pages, int n_pages, const float *__restrict__ slopes, const float *__restrict__ sinks,
    const float *__restrict__ gate, int ldg, void *__restrict__ out, int out_f32, int ldo, float *__restrict__ part_o,
    float2 *__restrict__ part_ml, int n_splits, int H, int Hkv, int Hv, int ldv, int heads_per_cta, int n_chunks, float scale, float softcap, int window,
    int keep_first, int *__restrict__ status) {
    pdl_trigger();
    pdl_wait();
    constexpr int D = KS * 16, DV = VS * 16;
    constexpr int LDK = D + 8, LDV = DV + 8;
    constexpr int WK = PAGE / DEC_WARPS;            // keys of a page per warp: 16
    constexpr int PW = WK + 8;                      // padded row of a warp's P^T (bfloat16)
    extern __shared__ __align__(16) uint8_t smem_raw[];
    constexpr size_t WARP_STAGE = (size_t)WK * (LDK + LDV);
    constexpr size_t WARP_BYTES = (STAGES * WARP_STAGE + NH * PW) * 2;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    __nv_bfloat16 *kv_w = reinterpret_cast<__nv_bfloat16 *>(smem_raw + (size_t)warp * WARP_BYTES);
    __nv_bfloat16 *Pw = kv_w + STAGES * WARP_STAGE;

    const int t = blockIdx.x;
    const int kvh = blockIdx.y / n_chunks, chunk = blockIdx.y - kvh * n_chunks;
    const int split = blockIdx.z;
    const int group = H / Hkv;
    const int h0 = kvh * group + chunk * heads_per_cta;
    const int g_count = min(heads_per_cta, group - chunk * heads_per_cta);
    const int mat = lane >> 3, mrow = lane & 7;
    const int pos = positions[t];
    const int *table = block_table + (size_t)seq_of_token[t] * max_blocks;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int n_pages_seq = pos / PAGE + 1;
    const int first_page = lo / PAGE;
    // the pages walked: those of the kept first tokens that lie before the window's, then the window's
    const int n_kp = window > 0 ? min((keep_first + PAGE - 1) / PAGE, first_page) : 0;
    const int n_walk = n_kp + n_pages_seq - first_page;
    const int pps = (n_walk + n_splits - 1) / n_splits;
    const int pb = split * pps;
    const int pe = min(pb + pps, n_walk);
    const int n_iter = max(pe - pb, 0);
    const int kvv = kvh / (Hkv / Hv);
    auto page_at = [&](int i) { return i < n_kp ? i : first_page + (i - n_kp); };
    const float LOG2E = 1.4426950408889634f;
    const float scale2 = scale * LOG2E;
    // this thread's two heads: columns (lane % 4) * 2 and + 1 of the S^T and O^T fragments
    float slope2[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int head = (lane & 3) * 2 + hh;
        slope2[hh] = (slopes && head < g_count) ? slopes[h0 + head] * LOG2E : 0.f;
    }

    auto load_rows = [&](int it) {
        const int pg = page_at(pb + it);
        const int page = pg < max_blocks ? table[pg] : -1;
        const bool have = page >= 0 && page < n_pages;
        if (!have && lane == 0) atomicExch(status, 3);
        const int valid_rows = have ? min(pos - pg * PAGE + 1, PAGE) : 0;
        const size_t cell = ((size_t)(have ? page : 0) * Hkv + kvh) * PAGE + (size_t)warp * WK;
        const size_t vcell = ((size_t)(have ? page : 0) * Hv + kvv) * PAGE + (size_t)warp * WK;
        __nv_bfloat16 *ks_ = kv_w + (size_t)(it % STAGES) * WARP_STAGE, *vs_ = ks_ + WK * LDK;
#pragma unroll
        for (int c = lane; c < WK * (D / 8); c += 32) {
            const int row = c / (D / 8), col = (c - row * (D / 8)) * 8;
            cp_async_16z(ks_ + row * LDK + col, k_pages + (cell + row) * D + col, warp * WK + row < valid_rows);
        }
#pragma unroll
        for (int c = lane; c < WK * (DV / 8); c += 32) {
            const int row = c / (DV / 8), col = (c - row * (DV / 8)) * 8;
            cp_async_16z(vs_ + row * LDV + col, v_pages + (vcell + row) * ldv + col, warp * WK + row < valid_rows);
        }
    };
#pragma unroll
    for (int it = 0; it < STAGES - 1; ++it) {
        if (it < n_iter) load_rows(it);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    // Q^T as B fragments: b0 holds (d = 16 ks + 2 (lane % 4) + {0, 1}, head = lane / 4), b1 the same 8 dims on
    uint32_t qb[KS][2];
    {
        const int head = lane >> 2;
        const __nv_bfloat16 *qrow = q + (size_t)t * ldq + (size_t)(h0 + head) * D + (lane & 3) * 2;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qb[ks][0] = head < g_count ? act_load(reinterpret_cast<const unsigned int *>(qrow + ks * 16)) : 0u;
            qb[ks][1] = head < g_count ? act_load(reinterpret_cast<const unsigned int *>(qrow + ks * 16 + 8)) : 0u;
        }
    }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float oacc[VS][4];
#pragma unroll
    for (int i = 0; i < VS; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;

    for (int it = 0; it < n_iter; ++it) {
        if (it + STAGES - 1 < n_iter) load_rows(it + STAGES - 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 1) : "memory");
        __syncwarp();
        const int pg = page_at(pb + it);
        const __nv_bfloat16 *ks_ = kv_w + (size_t)(it % STAGES) * WARP_STAGE, *vs_ = ks_ + WK * LDK;
        const int key_base = pg * PAGE + warp * WK;
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t a[4];
            ldmatrix_x4(a, ks_ + (size_t)((mat & 1) * 8 + mrow) * LDK + ks * 16 + (mat >> 1) * 8);
            mma_bf16(c, a, qb[ks][0], qb[ks][1]);
        }
        // rows of the fragment are keys (lane / 4, + 8), columns heads ((lane % 4) * 2, + 1)
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int kpos = key_base + (lane >> 2) + (i >> 1) * 8;
            c[i] = ((kpos >= lo || kpos < keep_first) && kpos <= pos)
                       ? (softcap > 0.f ? capped_score2(c[i], scale, softcap) : c[i] * scale2) - slope2[i & 1] * (float)(pos - kpos) : -INFINITY;
            mx[i & 1] = fmaxf(mx[i & 1], c[i]);
        }
        float corr[2];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 4));
            mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 8));
            mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 16));
            const float m_new = fmaxf(m_run[hh], mx[hh]);
            corr[hh] = (m_new == -INFINITY) ? 1.f : exp2f(m_run[hh] - m_new);
            m_run[hh] = m_new;
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int hh = i & 1;
            const float pf = (m_run[hh] == -INFINITY) ? 0.f : exp2f(c[i] - m_run[hh]);
            const __nv_bfloat16 ph = __float2bfloat16_rn(pf);
            l_run[hh] = (i < 2 ? l_run[hh] * corr[hh] : l_run[hh]) + __bfloat162float(ph);
            Pw[((lane & 3) * 2 + hh) * PW + (lane >> 2) + (i >> 1) * 8] = ph;
        }
        __syncwarp();
        const uint32_t pb0 = *reinterpret_cast<const uint32_t *>(Pw + (lane >> 2) * PW + (lane & 3) * 2);
        const uint32_t pb1 = *reinterpret_cast<const uint32_t *>(Pw + (lane >> 2) * PW + (lane & 3) * 2 + 8);
#pragma unroll
        for (int mt = 0; mt < VS; ++mt) {
            oacc[mt][0] *= corr[0];
            oacc[mt][1] *= corr[1];
            oacc[mt][2] *= corr[0];
            oacc[mt][3] *= corr[1];
            uint32_t a[4];
            ldmatrix_x4_trans(a, vs_ + (size_t)((mat >> 1) * 8 + mrow) * LDV + mt * 16 + (mat & 1) * 8);
            mma_bf16(oacc[mt], a, pb0, pb1);
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 4);
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 8);
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 16);
    }
    __syncthreads();                                             // every warp is done with its stages
    float *mo = reinterpret_cast<float *>(smem_raw);             // [WARPS][DV][NH] outputs, then [WARPS][NH] maxima and sums
    float *mm = mo + (size_t)DEC_WARPS * DV * NH, *ml = mm + DEC_WARPS * NH;
#pragma unroll
    for (int mt = 0; mt < VS; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int d = mt * 16 + (lane >> 2) + (i >> 1) * 8, head = (lane & 3) * 2 + (i & 1);
            mo[((size_t)warp * DV + d) * NH + head] = oacc[mt][i];
        }
    if (lane < 4) {
        mm[warp * NH + lane * 2] = m_run[0];
        mm[warp * NH + lane * 2 + 1] = m_run[1];
        ml[warp * NH + lane * 2] = l_run[0];
        ml[warp * NH + lane * 2 + 1] = l_run[1];
    }
    __syncthreads();
    for (int i = tid; i < DV * NH; i += DEC_WARPS * 32) {
        const int d = i / NH, head = i - d * NH;
        if (head >= g_count) continue;
        float m = -INFINITY;
        for (int w = 0; w < DEC_WARPS; ++w) m = fmaxf(m, mm[w * NH + head]);
        float o = 0.f, l = 0.f;
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float f = (mm[w * NH + head] == -INFINITY) ? 0.f : exp2f(mm[w * NH + head] - m);
            o += mo[((size_t)w * DV + d) * NH + head] * f;
            l += ml[w * NH + head] * f;
        }
        const int h = h0 + head;
        if (n_splits == 1) {
            const float sink2 = sinks ? sinks[h] * LOG2E : -INFINITY;
            const float m_all = fmaxf(m, sink2);
            const float f = (m == -INFINITY) ? 0.f : exp2f(m - m_all);
            const float den = l * f + (sinks ? exp2f(sink2 - m_all) : 0.f);
            float r = den > 0.f ? o * f / den : 0.f;
            if (gate) r *= 1.0f / (1.0f + __expf(-act_load(gate + (size_t)t * ldg + (size_t)h * DV + d)));
            store_out(out, out_f32, (size_t)t * ldo + (size_t)h * DV + d, r);
        } else {
            part_o[(((size_t)t * H + h) * n_splits + split) * DV + d] = o;
            if (d == 0) part_ml[((size_t)t * H + h) * n_splits + split] = make_float2(m, l);
        }
    }
}

template <int KS, int VS>
int launch_decode_mma(dim3 grid, cudaStream_t stream, const __nv_bfloat16 *q, int ldq, const int *positions, const int *seq_of_token,
                      const int *block_table, int max_blocks, const __nv_bfloat16 *k_pages, const __nv_bfloat16 *v_pages, int n_pages,
                      const float *slopes, const float *sinks, const float *gate, int ldg, void *out, int out_f32, int ldo, float *part_o,
                      float2 *part_ml, int n_splits, int H, int Hkv, int Hv, int ldv, int heads_per_cta, int n_chunks, float scale, float softcap, int window,
                      int keep_first, int *status) {
    constexpr int STAGES = 3;
    constexpr int D = KS * 16, DV = VS * 16;
    const size_t stages = (size_t)DEC_WARPS * ((size_t)STAGES * (PAGE / DEC_WARPS) * (D + 8 + DV + 8) + NH * (PAGE / DEC_WARPS + 8)) * 2;
    const size_t merge = sizeof(float) * ((size_t)DEC_WARPS * DV * NH + 2 * DEC_WARPS * NH);
    const size_t smem = stages > merge ? stages : merge;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(sink_decode_mma_kernel<KS, VS, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LGML_FAIL("sink_decode_mma: cannot have %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    lgml_launch(sink_decode_mma_kernel<KS, VS, STAGES>, grid, DEC_WARPS * 32, smem, stream, q, ldq, positions, seq_of_token, block_table, max_blocks,
                k_pages, v_pages, n_pages, slopes, sinks, gate, ldg, out, out_f32, ldo, part_o, part_ml, n_splits, H, Hkv, Hv, ldv, heads_per_cta,
                n_chunks, scale, softcap, window, keep_first, status);
    return lgml_launch_status("sink_decode_mma");
}

template <int GH, bool VEC>
int launch_decode(dim3 grid, size_t smem, cudaStream_t stream, const __nv_bfloat16 *q, int ldq, const int *positions, const int *seq_of_token,
                  const int *block_table, int max_blocks, const __nv_bfloat16 *k_pages, const __nv_bfloat16 *v_pages, int n_pages,
                  const float *slopes, const float *sinks, const float *gate, int ldg, void *out, int out_f32, int ldo, float *part_o,
                  float2 *part_ml, int n_splits, int n_chunks, int H, int Hkv, int Hv, int D, int Dv, int ldv, float scale, float softcap, int window,
                  int keep_first, int v_stage, int *status) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(sink_decode_kernel<GH, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LGML_FAIL("sink_decode: cannot have %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    }
    lgml_launch(sink_decode_kernel<GH, VEC>, grid, DEC_WARPS * 32, smem, stream, q, ldq, positions, seq_of_token, block_table, max_blocks, k_pages,
                v_pages, n_pages, slopes, sinks, gate, ldg, out, out_f32, ldo, part_o, part_ml, n_splits, n_chunks, H, Hkv, Hv, D, Dv, ldv, scale, softcap, window,
                keep_first, v_stage, status);
    return lgml_launch_status("sink_decode");
}
}  // namespace

// proj: float32 [n_tokens, ldp], columns q (H D) | k (Hkv D) | v (Hv Dv) | anything else.  Keys and values may have head
// counts of their own (several key heads that share one value head).
// v_keep: float32 [n_tokens, Hkv Dv], written (v_mode 1) or read (v_mode 2); v_lambda: one float32 on the device.
LGML_API int lgml_sink_qkv_store(const float *proj, int ldp, void *q_out, int dtype, int ldq, const int *positions, const int *seq_of_token,
                                 const int *block_table, int max_blocks, void *k_pages, void *v_pages, int n_pages, int page_size,
                                 int n_tokens, int H, int Hkv, int Hv, int D, int Dv, float temp_coef, int temp_every, int v_mode, float *v_keep,
                                 const float *v_lambda, int write_kv, int *status, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && H > 0 && Hkv > 0 && Hv > 0 && D > 0 && Dv > 0 && page_size > 0 && max_blocks > 0, "sink_qkv_store: bad sizes");
    LGML_REQUIRE(ldp >= H * D + (write_kv ? Hkv * D + Hv * Dv : 0), "sink_qkv_store: row stride %d is below the q, k and v columns", ldp);
    LGML_REQUIRE(ldq >= H * D, "sink_qkv_store: q row stride %d is below H D = %d", ldq, H * D);
    LGML_REQUIRE(temp_coef == 0.f || temp_every > 0, "sink_qkv_store: the temperature's step must be positive");
    LGML_REQUIRE(v_mode >= 0 && v_mode <= 2, "sink_qkv_store: unknown value mode %d", v_mode);
    LGML_REQUIRE(v_mode == 0 || v_keep != nullptr, "sink_qkv_store: value mode %d needs the kept values", v_mode);
    LGML_REQUIRE(v_mode != 2 || v_lambda != nullptr, "sink_qkv_store: mixing needs its weight");
    if (n_tokens == 0) return 0;
    const int items = H * D + (write_kv ? Hkv * D + Hv * Dv : 0);
    dim3 grid(n_tokens, (items + ITEMS - 1) / ITEMS);
    if (dtype == LGML_F32)
        lgml_launch(sink_qkv_store_kernel<float>, grid, ITEMS, 0, stream, proj, ldp, (float *)q_out, ldq, positions, seq_of_token, block_table,
                    max_blocks, (float *)k_pages, (float *)v_pages, n_pages, page_size, H, Hkv, Hv, D, Dv, temp_coef, temp_every, v_mode, v_keep,
                    v_lambda, write_kv, status);
    else if (dtype == LGML_BF16)
        lgml_launch(sink_qkv_store_kernel<__nv_bfloat16>, grid, ITEMS, 0, stream, proj, ldp, (__nv_bfloat16 *)q_out, ldq, positions, seq_of_token,
                    block_table, max_blocks, (__nv_bfloat16 *)k_pages, (__nv_bfloat16 *)v_pages, n_pages, page_size, H, Hkv, Hv, D, Dv, temp_coef,
                    temp_every, v_mode, v_keep, v_lambda, write_kv, status);
    else
        LGML_FAIL("sink_qkv_store: unknown type %d", dtype);
    return lgml_launch_status("sink_qkv_store");
}

// slopes, sinks: float32 [H] or null (no bias, no sink); gate: float32 [n_tokens, ldg] (column h Dv + d) or null.
// Hv value heads (Hkv a multiple of it: key heads g Hkv / Hv ... share value head g), value rows ldv elements apart
// (values that are a column range of wider cells), keep_first: the first tokens of a request that stay visible
// beyond the window; out_dtype: the output's type (float32 for a caller that combines heads afterwards).
LGML_API int lgml_sink_attention(const void *q, int dtype, int ldq, const int *positions, const int *seq_of_token, const int *block_table,
                                 int max_blocks, const void *k_pages, const void *v_pages, int n_pages, int page_size, const float *slopes,
                                 const float *sinks, const float *gate, int ldg, void *out, int out_dtype, int ldo, int n_tokens, int H, int Hkv,
                                 int Hv, int D, int Dv, int ldv, float scale, float softcap, int window, int keep_first, int *status, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && H > 0 && Hkv > 0 && Hv > 0 && D > 0 && Dv > 0 && page_size > 0 && max_blocks > 0, "sink_attention: bad sizes");
    LGML_REQUIRE(H % Hkv == 0, "sink_attention: %d heads are no multiple of %d KV heads", H, Hkv);
    LGML_REQUIRE(Hkv % Hv == 0, "sink_attention: %d key heads are no multiple of %d value heads", Hkv, Hv);
    LGML_REQUIRE(D <= GEN_MAX_D && Dv <= GEN_MAX_D, "sink_attention: head sizes %d and %d must be at most %d", D, Dv, GEN_MAX_D);
    LGML_REQUIRE(ldv >= Dv, "sink_attention: value rows %d apart hold no %d values", ldv, Dv);
    LGML_REQUIRE(H <= 65535, "sink_attention: too many heads");
    LGML_REQUIRE(window >= 0 && keep_first >= 0, "sink_attention: bad window");
    LGML_REQUIRE(gate == nullptr || ldg >= H * Dv, "sink_attention: the gate's row stride %d is below H Dv", ldg);
    LGML_REQUIRE(out_dtype == dtype || out_dtype == LGML_F32, "sink_attention: the output is the inputs' type or float32");
    if (n_tokens == 0) return 0;
    dim3 grid(n_tokens, H);
    if (dtype == LGML_F32)
        lgml_launch(sink_attention_kernel<float, float>, grid, WARPS * 32, 0, stream, (const float *)q, ldq, positions, seq_of_token, block_table,
                    max_blocks, (const float *)k_pages, (const float *)v_pages, n_pages, page_size, slopes, sinks, gate, ldg, (float *)out, ldo, H,
                    Hkv, Hv, D, Dv, ldv, scale, softcap, window, keep_first, status);
    else if (dtype == LGML_BF16 && out_dtype == LGML_F32)
        lgml_launch(sink_attention_kernel<__nv_bfloat16, float>, grid, WARPS * 32, 0, stream, (const __nv_bfloat16 *)q, ldq, positions, seq_of_token,
                    block_table, max_blocks, (const __nv_bfloat16 *)k_pages, (const __nv_bfloat16 *)v_pages, n_pages, page_size, slopes, sinks,
                    gate, ldg, (float *)out, ldo, H, Hkv, Hv, D, Dv, ldv, scale, softcap, window, keep_first, status);
    else if (dtype == LGML_BF16)
        lgml_launch(sink_attention_kernel<__nv_bfloat16, __nv_bfloat16>, grid, WARPS * 32, 0, stream, (const __nv_bfloat16 *)q, ldq, positions, seq_of_token,
                    block_table, max_blocks, (const __nv_bfloat16 *)k_pages, (const __nv_bfloat16 *)v_pages, n_pages, page_size, slopes, sinks,
                    gate, ldg, (__nv_bfloat16 *)out, ldo, H, Hkv, Hv, D, Dv, ldv, scale, softcap, window, keep_first, status);
    else
        LGML_FAIL("sink_attention: unknown type %d", dtype);
    return lgml_launch_status("sink_attention");
}

// The tensor-core form for prompts and portions (bfloat16, pages of 64, head sizes up to 128).
// tiles: int32 [n_tiles, 4] rows (request row, first token row, tokens <= 64, 0), each within one request.
// Hv, ldv, keep_first, out_f32: as for lgml_sink_attention (out_f32 != 0: a float32 output).
LGML_API int lgml_sink_attention_mma(const void *q, int ldq, const int *positions, const int *tiles, int n_tiles, const int *block_table,
                                     int max_blocks, const void *k_pages, const void *v_pages, int n_pages, int page_size,
                                     const float *slopes, const float *sinks, const float *gate, int ldg, void *out, int out_f32, int ldo, int H,
                                     int Hkv, int Hv, int D, int Dv, int ldv, float scale, float softcap, int window, int keep_first, int *status,
                                     cudaStream_t stream) {
    LGML_REQUIRE(n_tiles >= 0 && H > 0 && Hkv > 0 && Hv > 0 && D > 0 && Dv > 0 && max_blocks > 0, "sink_attention_mma: bad sizes");
    LGML_REQUIRE(Hkv % Hv == 0 && ldv >= Dv && keep_first >= 0, "sink_attention_mma: %d key heads on %d value heads, value rows %d apart", Hkv, Hv, ldv);
    LGML_REQUIRE(page_size == PAGE, "sink_attention_mma: pages of %d tokens, this kernel takes %d", page_size, PAGE);
    LGML_REQUIRE(H % Hkv == 0 && H <= 65535, "sink_attention_mma: %d heads on %d KV heads", H, Hkv);
    LGML_REQUIRE(D <= 128 && Dv <= 128, "sink_attention_mma: head sizes %d and %d must be at most 128", D, Dv);
    LGML_REQUIRE(window >= 0, "sink_attention_mma: bad window");
    LGML_REQUIRE(gate == nullptr || ldg >= H * Dv, "sink_attention_mma: the gate's row stride %d is below H Dv", ldg);
    if (n_tiles == 0) return 0;
    dim3 grid(n_tiles, H);
    const int ks = D <= 32 ? 2 : D <= 64 ? 4 : D <= 96 ? 6 : 8;
    const int nv = Dv <= 32 ? 4 : Dv <= 64 ? 8 : Dv <= 96 ? 12 : 16;
#define LGML_MMA_ARGS grid, stream, (const __nv_bfloat16 *)q, ldq, positions, tiles, block_table, max_blocks, (const __nv_bfloat16 *)k_pages, \
                      (const __nv_bfloat16 *)v_pages, n_pages, slopes, sinks, gate, ldg, out, out_f32, ldo, H, Hkv, Hv, D, Dv, ldv, scale, softcap, window, \
                      keep_first, status
#define LGML_MMA_NV(KK) \
    switch (nv) { case 4: return launch_mma<KK, 4>(LGML_MMA_ARGS); case 8: return launch_mma<KK, 8>(LGML_MMA_ARGS); \
                  case 12: return launch_mma<KK, 12>(LGML_MMA_ARGS); default: return launch_mma<KK, 16>(LGML_MMA_ARGS); }
    switch (ks) {
        case 2: LGML_MMA_NV(2)
        case 4: LGML_MMA_NV(4)
        case 6: LGML_MMA_NV(6)
        default: LGML_MMA_NV(8)
    }
#undef LGML_MMA_NV
#undef LGML_MMA_ARGS
}

// The split form for decoding and short portions (bfloat16, pages of 64, head sizes up to 256).
// scratch (float32, n_tokens H n_splits (Dv + 2) elements) is needed when n_splits > 1.
// Hv, ldv, keep_first, out_f32: as for lgml_sink_attention (out_f32 != 0: a float32 output).
LGML_API int lgml_sink_decode(const void *q, int ldq, const int *positions, const int *seq_of_token, const int *block_table, int max_blocks,
                              const void *k_pages, const void *v_pages, int n_pages, int page_size, const float *slopes, const float *sinks,
                              const float *gate, int ldg, void *out, int out_f32, int ldo, float *scratch, int n_splits, int n_tokens, int H,
                              int Hkv, int Hv, int D, int Dv, int ldv, float scale, float softcap, int window, int keep_first, int *status, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && H > 0 && Hkv > 0 && Hv > 0 && D > 0 && Dv > 0 && max_blocks > 0, "sink_decode: bad sizes");
    LGML_REQUIRE(Hkv % Hv == 0 && ldv >= Dv && keep_first >= 0, "sink_decode: %d key heads on %d value heads, value rows %d apart", Hkv, Hv, ldv);
    LGML_REQUIRE(page_size == PAGE, "sink_decode: pages of %d tokens, this kernel takes %d", page_size, PAGE);
    LGML_REQUIRE(H % Hkv == 0, "sink_decode: %d heads are no multiple of %d KV heads", H, Hkv);
    LGML_REQUIRE(D <= MAX_D && Dv <= MAX_D, "sink_decode: head sizes %d and %d must be at most %d", D, Dv, MAX_D);
    LGML_REQUIRE(n_splits >= 1 && n_splits <= DEC_MAX_SPLITS, "sink_decode: %d key ranges (1 to %d)", n_splits, DEC_MAX_SPLITS);
    LGML_REQUIRE(n_splits == 1 || scratch != nullptr, "sink_decode: %d ranges need scratch memory", n_splits);
    LGML_REQUIRE(window >= 0, "sink_decode: bad window");
    LGML_REQUIRE(gate == nullptr || ldg >= H * Dv, "sink_decode: the gate's row stride %d is below H Dv", ldg);
    if (n_tokens == 0) return 0;
    const int group = H / Hkv;
    float *part_o = scratch;
    float2 *part_ml = reinterpret_cast<float2 *>(scratch + (size_t)n_tokens * H * n_splits * Dv);
    if (D % 32 == 0 && Dv % 32 == 0 && D <= 128 && Dv <= 128 && ldq % 2 == 0 && ldv % 8 == 0 && (((uintptr_t)k_pages | (uintptr_t)v_pages) & 15) == 0 &&
        ((uintptr_t)q & 3) == 0) {
        // head sizes the tensor-core form is built for
        const int n_chunks = (group + NH - 1) / NH;
        const int heads_per_cta = (group + n_chunks - 1) / n_chunks;
        LGML_REQUIRE((long long)Hkv * n_chunks <= 65535, "sink_decode: too many heads");
        dim3 grid(n_tokens, Hkv * n_chunks, n_splits);
        int rc = 0;
#define LGML_DM_ARGS grid, stream, (const __nv_bfloat16 *)q, ldq, positions, seq_of_token, block_table, max_blocks, (const __nv_bfloat16 *)k_pages, \
                     (const __nv_bfloat16 *)v_pages, n_pages, slopes, sinks, gate, ldg, out, out_f32, ldo, part_o, part_ml, n_splits, H, Hkv, Hv, ldv, \
                     heads_per_cta, n_chunks, scale, softcap, window, keep_first, status
#define LGML_DM_VS(KK) \
    switch (Dv / 16) { case 2: rc = launch_decode_mma<KK, 2>(LGML_DM_ARGS); break; case 4: rc = launch_decode_mma<KK, 4>(LGML_DM_ARGS); break; \
                       case 6: rc = launch_decode_mma<KK, 6>(LGML_DM_ARGS); break; default: rc = launch_decode_mma<KK, 8>(LGML_DM_ARGS); break; } \
    break;
        switch (D / 16) {
            case 2: LGML_DM_VS(2)
            case 4: LGML_DM_VS(4)
            case 6: LGML_DM_VS(6)
            default: LGML_DM_VS(8)
        }
#undef LGML_DM_VS
#undef LGML_DM_ARGS
        if (rc || n_splits == 1) return rc;
        lgml_launch(sink_decode_combine_kernel, dim3(n_tokens, H), 128, 0, stream, (const float *)part_o, (const float2 *)part_ml, sinks, gate, ldg,
                    out, out_f32, ldo, n_splits, H, Dv);
        return lgml_launch_status("sink_decode_combine");
    }
    const int gh = group >= 8 ? 8 : group >= 4 ? 4 : group >= 2 ? 2 : 1;       // heads a CTA scores together
    const int n_chunks = (group + gh - 1) / gh;
    LGML_REQUIRE((long long)Hkv * n_chunks <= 65535, "sink_decode: too many heads");
    const bool vec = D % 8 == 0 && Dv % 4 == 0 && ldv % 8 == 0 && (((uintptr_t)k_pages | (uintptr_t)v_pages) & 15) == 0;
    // the values of a block go through shared memory when their rows are whole 16-byte pieces (and the floats before them keep that alignment)
    const int v_stage = vec && Dv % 8 == 0 && D % 4 == 0 && (size_t)DEC_WARPS * 32 * Dv * 2 <= 160 * 1024;
    const size_t smem = sizeof(float) * ((size_t)gh * D + (size_t)DEC_WARPS * gh * 32 + 2 * DEC_WARPS * gh + (size_t)DEC_WARPS * gh * Dv) +
                        (v_stage ? (size_t)DEC_WARPS * 32 * Dv * 2 : 0);
    dim3 grid(n_tokens, Hkv * n_chunks, n_splits);
    int rc;
#define LGML_DEC_ARGS grid, smem, stream, (const __nv_bfloat16 *)q, ldq, positions, seq_of_token, block_table, max_blocks, (const __nv_bfloat16 *)k_pages, \
                      (const __nv_bfloat16 *)v_pages, n_pages, slopes, sinks, gate, ldg, out, out_f32, ldo, part_o, part_ml, n_splits, n_chunks, H, \
                      Hkv, Hv, D, Dv, ldv, scale, softcap, window, keep_first, v_stage, status
#define LGML_DEC_GH(G) rc = vec ? launch_decode<G, true>(LGML_DEC_ARGS) : launch_decode<G, false>(LGML_DEC_ARGS); break;
    switch (gh) {
        case 8: LGML_DEC_GH(8)
        case 4: LGML_DEC_GH(4)
        case 2: LGML_DEC_GH(2)
        default: LGML_DEC_GH(1)
    }
#undef LGML_DEC_GH
#undef LGML_DEC_ARGS
    if (rc || n_splits == 1) return rc;
    lgml_launch(sink_decode_combine_kernel, dim3(n_tokens, H), 128, 0, stream, (const float *)part_o, (const float2 *)part_ml, sinks, gate, ldg,
                out, out_f32, ldo, n_splits, H, Dv);
    return lgml_launch_status("sink_decode_combine");
}
