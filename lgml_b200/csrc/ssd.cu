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
// Block: (column tile, head, request); a column's N entries are dealt over LN neighbouring lanes, RN each.
// The step's tokens come through shared memory in groups of TT: B, C, the tile's x, dt and the decay.
template <int RN>
__global__ void __launch_bounds__(SCAN_THREADS) ssd_scan_kernel(const float *__restrict__ xbc, int ldx, const float *__restrict__ dt_raw, int ldd,
                                                                const float *__restrict__ dt_bias, const float *__restrict__ a_log,
                                                                const float *__restrict__ d_skip, float *__restrict__ state, long long state_ld,
                                                                const int *__restrict__ seq_start, const int *__restrict__ slots,
                                                                float *__restrict__ y, int ldy, int Hs, int G, int P, int N, int LN, int TT) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float sm[];
    const int CPB = SCAN_THREADS / LN;
    float *Bs = sm, *Cs = Bs + (size_t)TT * N, *xs = Cs + (size_t)TT * N, *dts = xs + (size_t)TT * CPB, *dAs = dts + TT;
    const int h = blockIdx.y, s = blockIdx.z, g = h / (Hs / G);
    const int tid = threadIdx.x, col = tid / LN, ln = tid - col * LN;
    const int p = blockIdx.x * CPB + col;
    const int n0 = ln * RN;
    const int t0 = seq_start[s], t1 = seq_start[s + 1];
    const int x_cols = Hs * P;
    const float a = expf(__ldg(a_log + h)), bias = __ldg(dt_bias + h), dsk = __ldg(d_skip + h);
    float *st = state + (size_t)slots[s] * state_ld + ((size_t)h * P + (p < P ? p : 0)) * N + n0;
    float S[RN];
#pragma unroll
    for (int i = 0; i < RN; ++i) S[i] = (p < P && n0 + i < N) ? act_load(st + i) : 0.f;
    for (int tb = t0; tb < t1; tb += TT) {
        const int nt = min(TT, t1 - tb);
        __syncthreads();
        for (int i = tid; i < nt * N; i += SCAN_THREADS) {
            const int k = i / N, c = i - k * N;
            const float *rowp = xbc + (size_t)(tb + k) * ldx + x_cols;
            Bs[(size_t)k * N + c] = act_load(rowp + (size_t)g * N + c);
            Cs[(size_t)k * N + c] = act_load(rowp + (size_t)(G + g) * N + c);
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
            const float xv = xs[k * CPB + col], dA = dAs[k], dx = dts[k] * xv;
            const float *Bk = Bs + (size_t)k * N + n0, *Ck = Cs + (size_t)k * N + n0;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < RN; ++i) {
                if (n0 + i < N) {
                    S[i] = fmaf(dA, S[i], dx * Bk[i]);
                    acc = fmaf(S[i], Ck[i], acc);
                }
            }
            for (int o = LN >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (ln == 0 && p < P) y[(size_t)(tb + k) * ldy + (size_t)h * P + p] = fmaf(dsk, xv, acc);
        }
    }
    if (p < P) {
#pragma unroll
        for (int i = 0; i < RN; ++i)
            if (n0 + i < N) st[i] = S[i];
    }
}

// out[t, c] = (y[t, c] silu(z[t, c])) / rms over c's part * w[c]; block (token, part)
template <typename TO>
__global__ void __launch_bounds__(256) ssd_gate_norm_kernel(const float *__restrict__ y, int ldy, const float *__restrict__ z, int ldz,
                                                            const float *__restrict__ w, TO *__restrict__ out, int ldo, int part, float eps) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const int t = blockIdx.x, c0 = blockIdx.y * part;
    const float *yr = y + (size_t)t * ldy + c0, *zr = z + (size_t)t * ldz + c0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < part; i += 256) {
        const float v = act_load(yr + i) * silu_(act_load(zr + i));
        ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)part + eps);
    TO *orow = out + (size_t)t * ldo + c0;
    for (int i = threadIdx.x; i < part; i += 256) {
        const float v = act_load(yr + i) * silu_(act_load(zr + i));
        orow[i] = from_f32<TO>(v * inv * __ldg(w + c0 + i));
    }
}

}  // namespace

LGML_API int lgml_ssd_scan(const float *xbc, int ldx, const float *dt_raw, int ldd, const float *dt_bias, const float *a_log, const float *d_skip,
                           float *state, long long state_ld, const int *seq_start, const int *slots, float *y, int ldy, int n_seqs, int Hs, int G,
                           int P, int N, cudaStream_t stream) {
    LGML_REQUIRE(n_seqs >= 0 && Hs > 0 && G > 0 && P > 0 && N > 0, "ssd_scan: bad sizes");
    LGML_REQUIRE(Hs % G == 0, "ssd_scan: %d heads are no multiple of %d groups", Hs, G);
    LGML_REQUIRE(N <= 1024, "ssd_scan: a state of %d numbers per column is more than 1024", N);
    LGML_REQUIRE(state_ld >= (long long)Hs * P * N, "ssd_scan: the state's rows do not hold %d x %d x %d floats", Hs, P, N);
    LGML_REQUIRE(ldx >= Hs * P + 2 * G * N && ldd >= Hs && ldy >= Hs * P, "ssd_scan: rows too short");
    LGML_REQUIRE(n_seqs <= 65535 && Hs <= 65535, "ssd_scan: too many requests or heads");
    if (n_seqs == 0) return 0;
    // RN entries a lane, LN lanes a column (a power of two up to 32): the pair that wastes least, then the smaller RN
    static const int rns[5] = {8, 12, 16, 24, 32};
    int best_rn = 32, best_ln = 32, best_cover = 1 << 30;
    for (int i = 0; i < 5; ++i) {
        int ln = 1;
        while (ln * rns[i] < N && ln < 32) ln *= 2;
        if (ln * rns[i] < N) continue;
        if (ln * rns[i] < best_cover) best_cover = ln * rns[i], best_rn = rns[i], best_ln = ln;
    }
    const int LN = best_ln, CPB = SCAN_THREADS / LN;
    int TT = 16;
    while (TT > 1 && (size_t)TT * (2 * N + CPB + 2) * sizeof(float) > 40 * 1024) TT /= 2;
    const size_t smem = (size_t)TT * (2 * N + CPB + 2) * sizeof(float);
    dim3 grid((P + CPB - 1) / CPB, Hs, n_seqs);
#define LGML_SCAN(RN) lgml_launch(ssd_scan_kernel<RN>, grid, SCAN_THREADS, smem, stream, xbc, ldx, dt_raw, ldd, dt_bias, a_log, d_skip, state, \
                                  state_ld, seq_start, slots, y, ldy, Hs, G, P, N, LN, TT)
    switch (best_rn) {
        case 8: LGML_SCAN(8); break;
        case 12: LGML_SCAN(12); break;
        case 16: LGML_SCAN(16); break;
        case 24: LGML_SCAN(24); break;
        default: LGML_SCAN(32); break;
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
    if (out_dtype == LGML_F32)
        lgml_launch(ssd_gate_norm_kernel<float>, grid, 256, 0, stream, y, ldy, z, ldz, w, (float *)out, ldo, part, eps);
    else if (out_dtype == LGML_BF16)
        lgml_launch(ssd_gate_norm_kernel<__nv_bfloat16>, grid, 256, 0, stream, y, ldy, z, ldz, w, (__nv_bfloat16 *)out, ldo, part, eps);
    else
        LGML_FAIL("ssd_gate_norm: unknown output type %d", out_dtype);
    return lgml_launch_status("ssd_gate_norm");
}
