// A selective state-space recurrence with a scalar decay per head ("state-space duality"):
//
//   dt_t = softplus(dt_raw_t + dt_bias_h)                       per head h
//   S_t  = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t B_t x_t^T      S is [N, P] per head; B, C are shared by the heads of a group
//   y_t  = S_t^T C_t + D_h x_t
//
//   ssd_scan       the recurrence over a step's tokens, request by request, S in the request's state slot
//   ssd_gate_norm  (y silu(z)) over the root mean square of each of `groups` equal parts, times a weight
//
// Everything is float32 arithmetic in both compute types.  The state of a head is stored column by
// column ([P][N]): a thread owns a slice of one column and keeps it in registers over the step's tokens.
#include <math.h>

#include "common.cuh"

LGML_DEFINE_LAST_ERROR(lgml_ssd)

namespace {

constexpr int SCAN_THREADS = 128;

__device__ __forceinline__ float softplus_(float v) { return v > 20.f ? v : log1pf(expf(v)); }
__device__ __forceinline__ float silu_(float v) { return v / (1.0f + expf(-v)); }

// xbc float32 [n, ldx]: x of head h at column h P, B of group g at column x_cols + g N, C at x_cols + (G + g) N.
// dt_raw float32 [n, ldd], column h.  state: per slot [Hs][P][N].  y float32 [n, ldy], column h P + p.
// Block: (column tile, head, request).  A thread owns RN entries of each of CQ neighbouring columns: what it reads of
// a token's B and C serves CQ columns (the shared-memory reads are what bounds this kernel).  A column's N entries are
// dealt over LN neighbouring lanes in groups of four: lane l owns the groups l, l + LN, l + 2 LN ..., so the lanes
// read neighbouring 16-byte pieces of B and C from shared memory (no bank is asked twice) and of the state from memory.
// The step's tokens come through shared memory in groups of TT: B, C (rows of NS = LN RN floats, zeros behind N),
// the tile's x, dt and the decay.
template <int RN, int CQ>
__global__ void __launch_bounds__(SCAN_THREADS) ssd_scan_kernel(const float *__restrict__ xbc, int ldx, const float *__restrict__ dt_raw, int ldd,
                                                                const float *__restrict__ dt_bias, const float *__restrict__ a_log,
                                                                const float *__restrict__ d_skip, float *__restrict__ state, long long state_ld,
                                                                const int *__restrict__ seq_start, const int *__restrict__ slots,
                                                                float *__restrict__ y, int ldy, int Hs, int G, int P, int N, int LN, int TT,
                                                                int pieces, int zero_start, float *__restrict__ decay_out, int vec) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float sm[];
    const int CPB = (SCAN_THREADS / LN) * CQ;          // columns of a block
    const int NS = LN * RN;
    float *Bs = sm, *Cs = Bs + (size_t)TT * NS, *xs = Cs + (size_t)TT * NS, *dts = xs + (size_t)TT * CPB, *dAs = dts + TT;
    const int h = blockIdx.y, s = blockIdx.z, g = h / (Hs / G);
    const int tid = threadIdx.x, col = tid / LN, ln = tid - col * LN;
    const int p0 = blockIdx.x * CPB + col * CQ;        // this thread's first column
    auto n_of = [&](int i) { return ((i >> 2) * LN + ln) * 4 + (i & 3); };      // the state entry behind this lane's i-th register
    // pieces: the step's tokens in pieces of consecutive tokens, rows (first, past the last) of an [n, 2] table
    const int t0 = pieces ? seq_start[2 * s] : seq_start[s], t1 = pieces ? seq_start[2 * s + 1] : seq_start[s + 1];
    const int x_cols = Hs * P;
    const float a = expf(__ldg(a_log + h)), bias = __ldg(dt_bias + h), dsk = __ldg(d_skip + h);
    float *st = state + (size_t)(slots ? slots[s] : s) * state_ld + (size_t)h * P * N;
    float S[CQ][RN];
#pragma unroll
    for (int q = 0; q < CQ; ++q)
#pragma unroll
        for (int i = 0; i < RN; ++i) S[q][i] = (!zero_start && p0 + q < P && n_of(i) < N) ? act_load(st + (size_t)(p0 + q) * N + n_of(i)) : 0.f;
    float decay = 1.f;
    const bool want_y = y != nullptr;
    for (int tb = t0; tb < t1; tb += TT) {
        const int nt = min(TT, t1 - tb);
        __syncthreads();
        if (vec) {
            // 16 bytes a load, the loads of four rounds in flight before the first is stored
            const int NS4 = NS >> 2, N4 = N >> 2, total = nt * NS4;
            for (int i0 = tid; i0 < total; i0 += 4 * SCAN_THREADS) {
                float4 vb[4], vc[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i = i0 + u * SCAN_THREADS;
                    vb[u] = vc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (i < total) {
                        const int k = i / NS4, c = i - k * NS4;
                        if (c < N4) {
                            const float *rowp = xbc + (size_t)(tb + k) * ldx + x_cols;
                            vb[u] = act_load(reinterpret_cast<const float4 *>(rowp + (size_t)g * N) + c);
                            vc[u] = act_load(reinterpret_cast<const float4 *>(rowp + (size_t)(G + g) * N) + c);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i = i0 + u * SCAN_THREADS;
                    if (i < total) reinterpret_cast<float4 *>(Bs)[i] = vb[u], reinterpret_cast<float4 *>(Cs)[i] = vc[u];
                }
            }
        } else {
            for (int i = tid; i < nt * NS; i += SCAN_THREADS) {
                const int k = i / NS, c = i - k * NS;
                const float *rowp = xbc + (size_t)(tb + k) * ldx + x_cols;
                Bs[i] = c < N ? act_load(rowp + (size_t)g * N + c) : 0.f;
                Cs[i] = c < N ? act_load(rowp + (size_t)(G + g) * N + c) : 0.f;
            }
        }
        for (int i = tid; i < nt * CPB; i += SCAN_THREADS) {
            const int k = i / CPB, c = i - k * CPB;
            const int pc = blockIdx.x * CPB + c;
            xs[k * CPB + c] = pc < P ? act_load(xbc + (size_t)(tb + k) * ldx + (size_t)h * P + pc) : 0.f;
        }
        for (int k = tid; k < nt; k += SCAN_THREADS) {
            const float dt = softplus_(act_load(dt_raw + (size_t)(tb + k) * ldd + h) + bias);
            dts[k] = dt;
            dAs[k] = expf(-a * dt);
        }
        __syncthreads();
        for (int k = 0; k < nt; ++k) {
            const float dA = dAs[k], dt = dts[k];
            float xv[CQ], dx[CQ], acc[CQ];
#pragma unroll
            for (int q = 0; q < CQ; ++q) xv[q] = xs[k * CPB + col * CQ + q], dx[q] = dt * xv[q], acc[q] = 0.f;
            decay *= dA;
            const float4 *Bk = reinterpret_cast<const float4 *>(Bs + (size_t)k * NS) + ln, *Ck = reinterpret_cast<const float4 *>(Cs + (size_t)k * NS) + ln;
#pragma unroll
            for (int j = 0; j < RN / 4; ++j) {
                const float4 b = Bk[j * LN];
#pragma unroll
                for (int q = 0; q < CQ; ++q) {
                    S[q][4 * j] = fmaf(dA, S[q][4 * j], dx[q] * b.x), S[q][4 * j + 1] = fmaf(dA, S[q][4 * j + 1], dx[q] * b.y);
                    S[q][4 * j + 2] = fmaf(dA, S[q][4 * j + 2], dx[q] * b.z), S[q][4 * j + 3] = fmaf(dA, S[q][4 * j + 3], dx[q] * b.w);
                }
                if (want_y) {
                    const float4 c = Ck[j * LN];
#pragma unroll
                    for (int q = 0; q < CQ; ++q) {
                        acc[q] = fmaf(S[q][4 * j], c.x, acc[q]), acc[q] = fmaf(S[q][4 * j + 1], c.y, acc[q]);
                        acc[q] = fmaf(S[q][4 * j + 2], c.z, acc[q]), acc[q] = fmaf(S[q][4 * j + 3], c.w, acc[q]);
                    }
                }
            }
            if (want_y) {
#pragma unroll
                for (int q = 0; q < CQ; ++q) {
                    for (int o = LN >> 1; o > 0; o >>= 1) acc[q] += __shfl_xor_sync(0xffffffffu, acc[q], o);
                    if (ln == 0 && p0 + q < P) y[(size_t)(tb + k) * ldy + (size_t)h * P + p0 + q] = fmaf(dsk, xv[q], acc[q]);
                }
            }
        }
    }
#pragma unroll
    for (int q = 0; q < CQ; ++q)
        if (p0 + q < P) {
#pragma unroll
            for (int i = 0; i < RN; ++i)
                if (n_of(i) < N) st[(size_t)(p0 + q) * N + n_of(i)] = S[q][i];
        }
    if (decay_out != nullptr && blockIdx.x == 0 && tid == 0) decay_out[(size_t)s * Hs + h] = decay;
}

// The chain over a request's pieces: scratch[c] holds what piece c's scan from zero left; it becomes the state piece c
// starts from, S_start(c + 1) = decay(c) S_start(c) + left(c); the request's slot gives the first start and takes the
// last end.  One thread per float of the state, the pieces of a request in order.
__global__ void __launch_bounds__(256) ssd_chain_kernel(float *__restrict__ scratch, long long scratch_ld, const float *__restrict__ decay,
                                                        float *__restrict__ state, long long state_ld, const int *__restrict__ first_piece,
                                                        const int *__restrict__ slots, int Hs, int PN) {
    pdl_trigger();
    pdl_wait();
    const int s = blockIdx.y;
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= Hs * PN) return;
    const int h = i / PN;
    float *st = state + (size_t)slots[s] * state_ld + i;
    float S = act_load(st);
    const int c0 = first_piece[s], c1 = first_piece[s + 1];
    constexpr int AHEAD = 8;            // the loads of eight pieces are in flight before the first is used
    for (int c = c0; c < c1; c += AHEAD) {
        float left[AHEAD], d[AHEAD];
#pragma unroll
        for (int u = 0; u < AHEAD; ++u)
            if (c + u < c1) left[u] = act_load(scratch + (size_t)(c + u) * scratch_ld + i), d[u] = act_load(decay + (size_t)(c + u) * Hs + h);
#pragma unroll
        for (int u = 0; u < AHEAD; ++u)
            if (c + u < c1) {
                scratch[(size_t)(c + u) * scratch_ld + i] = S;
                S = fmaf(d[u], S, left[u]);
            }
    }
    *st = S;
}

// out[t, c] = (y[t, c] silu(z[t, c])) / rms over c's part * w[c]; block (token, part).  The gated values wait in shared
// memory between the sum of squares and the division when a part fits there (keep != 0): y and z are then read once.
template <typename TO, int NT>
__global__ void __launch_bounds__(NT) ssd_gate_norm_kernel(const float *__restrict__ y, int ldy, const float *__restrict__ z, int ldz,
                                                             const float *__restrict__ w, TO *__restrict__ out, int ldo, int part, float eps, int keep) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float gated[];
    __shared__ float red[32];
    const int t = blockIdx.x, c0 = blockIdx.y * part;
    const float *yr = y + (size_t)t * ldy + c0, *zr = z + (size_t)t * ldz + c0;
    float ss = 0.f;
#pragma unroll 4
    for (int i = threadIdx.x; i < part; i += NT) {
        const float v = act_load(yr + i) * silu_(act_load(zr + i));
        if (keep) gated[i] = v;
        ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)part + eps);
    TO *orow = out + (size_t)t * ldo + c0;
#pragma unroll 4
    for (int i = threadIdx.x; i < part; i += NT) {
        const float v = keep ? gated[i] : act_load(yr + i) * silu_(act_load(zr + i));
        orow[i] = from_f32<TO>(v * inv * __ldg(w + c0 + i));
    }
}

}  // namespace

LGML_API int lgml_ssd_scan(const float *xbc, int ldx, const float *dt_raw, int ldd, const float *dt_bias, const float *a_log, const float *d_skip,
                           float *state, long long state_ld, const int *seq_start, const int *slots, float *y, int ldy, int n_seqs, int Hs, int G,
                           int P, int N, int pieces, int zero_start, float *decay_out, cudaStream_t stream) {
    LGML_REQUIRE(n_seqs >= 0 && Hs > 0 && G > 0 && P > 0 && N > 0, "ssd_scan: bad sizes");
    LGML_REQUIRE(Hs % G == 0, "ssd_scan: %d heads are no multiple of %d groups", Hs, G);
    LGML_REQUIRE(N <= 1024, "ssd_scan: a state of %d numbers per column is more than 1024", N);
    LGML_REQUIRE(state_ld >= (long long)Hs * P * N, "ssd_scan: the state's rows do not hold %d x %d x %d floats", Hs, P, N);
    LGML_REQUIRE(ldx >= Hs * P + 2 * G * N && ldd >= Hs && ldy >= Hs * P, "ssd_scan: rows too short");
    LGML_REQUIRE(n_seqs <= 65535 && Hs <= 65535, "ssd_scan: too many requests, pieces or heads");
    LGML_REQUIRE(slots != nullptr || pieces, "ssd_scan: requests come with their slots");
    if (n_seqs == 0) return 0;
    // RN entries a lane, LN lanes a column (a power of two up to 32): the pair that wastes least, then the smaller RN.
    // Four columns a thread with up to 16 entries each (states up to 512 numbers a column), else one column with up to 32.
    const bool quad = N <= 512;
    static const int rns[6] = {4, 8, 12, 16, 24, 32};
    int best_rn = 32, best_ln = 32, best_cover = 1 << 30;
    for (int i = 0; i < 6; ++i) {
        if (quad ? rns[i] > 16 : rns[i] < 8) continue;
        int ln = 1;
        while (ln * rns[i] < N && ln < 32) ln *= 2;
        if (ln * rns[i] < N) continue;
        // (at equal cover: with four columns a thread the larger RN, fewer lanes to add up; with one the smaller, more threads)
        if (ln * rns[i] < best_cover || (quad && ln * rns[i] == best_cover)) best_cover = ln * rns[i], best_rn = rns[i], best_ln = ln;
    }
    const int LN = best_ln, CQ = quad ? 4 : 1, CPB = (SCAN_THREADS / LN) * CQ;
    const int NS = LN * best_rn;
    int TT = 32;
    while (TT > 1 && (size_t)TT * (2 * NS + CPB + 2) * sizeof(float) > 46 * 1024) TT /= 2;
    const size_t smem = (size_t)TT * (2 * NS + CPB + 2) * sizeof(float);
    dim3 grid((P + CPB - 1) / CPB, Hs, n_seqs);
    const int vec = N % 4 == 0 && ldx % 4 == 0 && (Hs * P) % 4 == 0 && ((uintptr_t)xbc & 15) == 0;
#define LGML_SCAN(RN, CQ) lgml_launch(ssd_scan_kernel<RN, CQ>, grid, SCAN_THREADS, smem, stream, xbc, ldx, dt_raw, ldd, dt_bias, a_log, d_skip, state, \
                                      state_ld, seq_start, slots, y, ldy, Hs, G, P, N, LN, TT, pieces, zero_start, decay_out, vec)
    if (quad) {
        switch (best_rn) {
            case 4: LGML_SCAN(4, 4); break;
            case 8: LGML_SCAN(8, 4); break;
            case 12: LGML_SCAN(12, 4); break;
            default: LGML_SCAN(16, 4); break;
        }
    } else {
        switch (best_rn) {
            case 8: LGML_SCAN(8, 1); break;
            case 12: LGML_SCAN(12, 1); break;
            case 16: LGML_SCAN(16, 1); break;
            case 24: LGML_SCAN(24, 1); break;
            default: LGML_SCAN(32, 1); break;
        }
    }
#undef LGML_SCAN
    return lgml_launch_status("ssd_scan");
}

LGML_API int lgml_ssd_gate_norm(const float *y, int ldy, const float *z, int ldz, const float *w, void *out, int out_dtype, int ldo, int n_tokens,
                                int inner, int groups, float eps, cudaStream_t stream) {
    LGML_REQUIRE(n_tokens >= 0 && inner > 0 && groups > 0 && inner % groups == 0, "ssd_gate_norm: %d channels in %d parts", inner, groups);
    LGML_REQUIRE(ldy >= inner && ldz >= inner && ldo >= inner && groups <= 65535, "ssd_gate_norm: rows too short");
    if (n_tokens == 0) return 0;
    dim3 grid(n_tokens, groups);
    const int part = inner / groups;
    const int threads = (n_tokens * groups <= 296 && part >= 1024) ? 1024 : 256;      // few rows: more threads share a row's latency
    const int keep = (size_t)part * sizeof(float) <= 40 * 1024;
    const size_t smem = keep ? (size_t)part * sizeof(float) : 0;
#define LGML_GN(TO, NT) lgml_launch(ssd_gate_norm_kernel<TO, NT>, grid, NT, smem, stream, y, ldy, z, ldz, w, (TO *)out, ldo, part, eps, keep)
    if (out_dtype == LGML_F32) { if (threads == 1024) LGML_GN(float, 1024); else LGML_GN(float, 256); }
    else if (out_dtype == LGML_BF16) { if (threads == 1024) LGML_GN(__nv_bfloat16, 1024); else LGML_GN(__nv_bfloat16, 256); }
    else LGML_FAIL("ssd_gate_norm: unknown output type %d", out_dtype);
#undef LGML_GN
    return lgml_launch_status("ssd_gate_norm");
}

// See ssd_chain_kernel.  scratch: [pieces, >= Hs P N]; decay: [pieces, Hs]; first_piece: [n_seqs + 1].
LGML_API int lgml_ssd_chain(float *scratch, long long scratch_ld, const float *decay, float *state, long long state_ld, const int *first_piece,
                            const int *slots, int n_seqs, int Hs, int P, int N, cudaStream_t stream) {
    LGML_REQUIRE(n_seqs >= 0 && Hs > 0 && P > 0 && N > 0 && n_seqs <= 65535, "ssd_chain: bad sizes");
    LGML_REQUIRE(scratch_ld >= (long long)Hs * P * N && state_ld >= (long long)Hs * P * N, "ssd_chain: rows too short");
    if (n_seqs == 0) return 0;
    dim3 grid((Hs * P * N + 255) / 256, n_seqs);
    lgml_launch(ssd_chain_kernel, grid, 256, 0, stream, scratch, scratch_ld, decay, state, state_ld, first_piece, slots, Hs, P * N);
    return lgml_launch_status("ssd_chain");
}
