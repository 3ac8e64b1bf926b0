// Gated delta rule behind short causal convolutions: a matrix state per head that decays, is corrected towards the
// current value along the current key and is read with the query.  Everything here is fp32.
//   prep  (one warp or block per head and rows):    convolutions + silu, unit-length q / k, their dot product, beta
//                                                   and decay of every head
//   rule  (sequential in time):  S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
// A sequence's state lives with its cache: two copies of the heads' matrices, column-major (a launch whose first token is at position
// p0 reads copy p0 & 1 and writes copy (p0 + n) & 1, so a step that is run twice leaves the same state) and a ring of
// the convolutions' last inputs (slot = position mod taps).
#include "common.h"
#include "ptx.cuh"

namespace b200 {

__device__ __forceinline__ float* delta_state(const b200_delta_args& a, int s) {
    float* base = a.state_ptrs ? reinterpret_cast<float*>(a.state_ptrs[(size_t)s * a.state_ptr_stride]) : a.state;
    return base + a.state_off;
}

__device__ __forceinline__ float softplus32(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

// ------------------------------------------------------------------ prep
// One block per (group of consecutive rows of a sequence, unit); a unit is a query head with its key head (convolved,
// activated, made unit vectors, and their dot product, which the read-out needs) or a value head (convolved and
// activated); the block of unit 0 also evaluates beta and the decay of every head.  Runs of tokens take one WARP per
// unit (the step is bound by instruction issue there: no barrier and no shared-memory reduction per row), a decode step
// four warps (its time is the chain of one row's loads).
template <int kPrepThreads>
__global__ void __launch_bounds__(kPrepThreads) delta_prep_kernel(b200_delta_args a, int rows_per_block) {
    extern __shared__ float y[];                   // pair: q [dim] | k [dim]; value head: [vdim]
    __shared__ float red[3][4];
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int unit = blockIdx.y, tid = threadIdx.x;
    const int groups = (a.seq_len + rows_per_block - 1) / rows_per_block;
    const int s = blockIdx.x / groups, i0 = (blockIdx.x - s * groups) * rows_per_block;
    const int i1 = i0 + rows_per_block < a.seq_len ? i0 + rows_per_block : a.seq_len;
    for (int i = i0; i < i1; ++i) {
    const int r = s * a.seq_len + i;
    if (kPrepThreads > 32)
        __syncthreads();                           // red is free again
    else
        __syncwarp();
    const int p = (a.pos ? a.pos[s] : a.pos0) + i;
    const int D = a.dim, V = a.vdim, G = a.kv_heads, H = a.heads;
    const int qk = G * D, C = 2 * qk + H * V, taps = a.taps;
    const float* ring = delta_state(a, s) + (size_t)2 * H * D * V;
    const float* row = a.proj + (size_t)r * a.ldp + a.c_off;
    float* out = a.work + (size_t)r * a.ldw;
    auto conv = [&](int c) {
        const float* w = a.conv_w + (size_t)c * taps;
        float acc = 0.f;
        if (i >= taps - 1) {                       // every input is a row of this launch (all but its first rows)
            for (int b = taps - 1; b >= 0; --b) acc = fmaf(w[taps - 1 - b], row[c - (ptrdiff_t)b * a.ldp], acc);
        } else {
            for (int b = taps - 1; b >= 0; --b) {  // oldest input first
                if (p - b < 0) continue;           // before the sequence's start: zero
                float x;
                if (b <= i)
                    x = row[c - (ptrdiff_t)b * a.ldp];
                else
                    x = ring[(size_t)((p - b) % taps) * C + c];
                acc = fmaf(w[taps - 1 - b], x, acc);
            }
        }
        return acc / (1.0f + expf(-acc));
    };
    if (unit == 0) {
        const float* rr = a.proj + (size_t)r * a.ldp;
        for (int h = tid; h < H; h += kPrepThreads) {
            out[C + h] = 1.0f / (1.0f + expf(-rr[a.b_off + h]));
            out[C + H + h] = expf(-expf(a.A_log[h]) * softplus32(rr[a.a_off + h] + a.dt_bias[h]));
        }
    }
    if (unit >= G) {                               // a value head
        const int h = unit - G;
        for (int d = tid; d < V; d += kPrepThreads) out[2 * qk + h * V + d] = conv(2 * qk + h * V + d);
        continue;
    }
    const int g = unit;
    float sq = 0.f, sk = 0.f;
    for (int d = tid; d < D; d += kPrepThreads) {
        const float qv = conv(g * D + d), kv = conv(qk + g * D + d);
        y[d] = qv;
        y[D + d] = kv;
        sq = fmaf(qv, qv, sq);
        sk = fmaf(kv, kv, sk);
    }
    float dot = 0.f;
    for (int d = tid; d < D; d += kPrepThreads) dot = fmaf(y[d], y[D + d], dot);   // (each thread reads what it wrote)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        sq += __shfl_xor_sync(0xffffffffu, sq, o);
        sk += __shfl_xor_sync(0xffffffffu, sk, o);
        dot += __shfl_xor_sync(0xffffffffu, dot, o);
    }
    if (kPrepThreads > 32) {
        if ((tid & 31) == 0) red[0][tid >> 5] = sq, red[1][tid >> 5] = sk, red[2][tid >> 5] = dot;
        __syncthreads();
        sq = sk = dot = 0.f;
#pragma unroll
        for (int w = 0; w < kPrepThreads / 32; ++w) sq += red[0][w], sk += red[1][w], dot += red[2][w];
    }
    const float fq = (1.0f / sqrtf(sq + a.unit_eps)) * rsqrtf((float)D), fk = 1.0f / sqrtf(sk + a.unit_eps);
    for (int d = tid; d < D; d += kPrepThreads) {
        out[g * D + d] = y[d] * fq;
        out[qk + g * D + d] = y[D + d] * fk;
    }
    if (tid == 0) out[C + 2 * H + g] = dot * fq * fk;
    }
}

// ------------------------------------------------------------------ rule
constexpr int kDeltaBatch = 16;      // most tokens staged in shared memory at a time (two buffers)

__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16f(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// Block = (sequence, head, NC * 256 / SL columns of S).  A group of SL lanes holds NC columns: column j's rows
// slice * NR .. + NR are in the registers of one lane, the dot products over a column meet by log2(SL) shuffles.  The
// NC columns of a group share every read of k and q and give the warp NC independent chains per token.  The state is
// kept column-major ([head][column][row]) so that a lane's rows are contiguous.  Tokens are staged 16 at a time by
// cp.async into one of two buffers while the other one is being consumed.
template <int NR, int SL, int NC>
__global__ void __launch_bounds__(256) delta_rule_kernel(b200_delta_args a, int vec, int tb) {
    extern __shared__ __align__(16) float sm[];
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    constexpr int Dp = NR * SL, COLS = NC * 256 / SL, CPW = 32 / SL;
    constexpr int STRIDE = 2 * Dp + COLS + 4;       // k | q | v columns | beta, decay, k.q, -
    const int s = blockIdx.x, h = blockIdx.y, tile = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int slice = lane % SL, cw = (warp * CPW + lane / SL) * NC, j = tile * COLS + cw;    // first column of the group
    const int D = a.dim, V = a.vdim, H = a.heads;
    const int g = h / (H / a.kv_heads);
    const int qk = a.kv_heads * D, C = 2 * qk + H * V;
    const int p0 = a.pos ? a.pos[s] : a.pos0;
    float* st = delta_state(a, s);
    float S[NC][NR];
#pragma unroll
    for (int c = 0; c < NC; ++c) {
        const float* src = st + (((size_t)(p0 & 1) * H + h) * V + j + c) * D;
#pragma unroll
        for (int n = 0; n < NR; ++n) {
            const int i = slice * NR + n;
            S[c][n] = (p0 > 0 && j + c < V && i < D) ? src[i] : 0.f;
        }
    }
    for (int e = tid; e < 2 * tb * STRIDE; e += 256) sm[e] = 0.f;               // rows beyond dim stay zero
    __syncthreads();
    const int tok = tid >> 4, sub = tid & 15;        // 16 threads stage one token
    auto stage = [&](int buf, int t0) {
        const int nb = a.seq_len - t0 < tb ? a.seq_len - t0 : tb;
        if (tok < nb) {
            const float* w = a.work + (size_t)(s * a.seq_len + t0 + tok) * a.ldw;
            float* dst = sm + (buf * tb + tok) * STRIDE;
            if (vec) {
                for (int c = sub * 4; c < D; c += 64) {
                    cp_async16f(dst + c, w + qk + g * D + c);
                    cp_async16f(dst + Dp + c, w + g * D + c);
                }
            } else {
                for (int c = sub; c < D; c += 16) {
                    cp_async4(dst + c, w + qk + g * D + c);
                    cp_async4(dst + Dp + c, w + g * D + c);
                }
            }
            for (int c = sub; c < COLS; c += 16)
                if (tile * COLS + c < V) cp_async4(dst + 2 * Dp + c, w + 2 * qk + h * V + tile * COLS + c);
            if (sub == 0) cp_async4(dst + 2 * Dp + COLS, w + C + h);
            if (sub == 1) cp_async4(dst + 2 * Dp + COLS + 1, w + C + H + h);
            if (sub == 2) cp_async4(dst + 2 * Dp + COLS + 2, w + C + 2 * H + g);
        }
        cp_commit();
    };
    stage(0, 0);
    int buf = 0;
    for (int t0 = 0; t0 < a.seq_len; t0 += tb, buf ^= 1) {
        const int nb = a.seq_len - t0 < tb ? a.seq_len - t0 : tb;
        if (t0 + tb < a.seq_len) {
            stage(buf ^ 1, t0 + tb);
            cp_wait<1>();
        } else {
            cp_wait<0>();
        }
        __syncthreads();
        for (int b = 0; b < nb; ++b) {
            const float* kk = sm + (buf * tb + b) * STRIDE + slice * NR;
            const float* qq = kk + Dp;
            const float* sc = sm + (buf * tb + b) * STRIDE + 2 * Dp;
            float kr[NR];
            float dk[NC], dq[NC];
#pragma unroll
            for (int c = 0; c < NC; ++c) dk[c] = dq[c] = 0.f;
#pragma unroll
            for (int n = 0; n < NR; n += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(kk + n);
                const float4 q4 = *reinterpret_cast<const float4*>(qq + n);
                kr[n] = k4.x, kr[n + 1] = k4.y, kr[n + 2] = k4.z, kr[n + 3] = k4.w;
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    dk[c] = fmaf(S[c][n], k4.x, dk[c]);
                    dq[c] = fmaf(S[c][n], q4.x, dq[c]);
                    dk[c] = fmaf(S[c][n + 1], k4.y, dk[c]);
                    dq[c] = fmaf(S[c][n + 1], q4.y, dq[c]);
                    dk[c] = fmaf(S[c][n + 2], k4.z, dk[c]);
                    dq[c] = fmaf(S[c][n + 2], q4.z, dq[c]);
                    dk[c] = fmaf(S[c][n + 3], k4.w, dk[c]);
                    dq[c] = fmaf(S[c][n + 3], q4.w, dq[c]);
                }
            }
            // both sums of a column in one butterfly: after the first exchange the even lanes carry S^T k, the odd
            // lanes S^T q (shuffles and shared-memory reads are what this loop is bound by)
            float mine[NC];
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                mine[c] = (lane & 1) ? dq[c] : dk[c];
                mine[c] += __shfl_xor_sync(0xffffffffu, (lane & 1) ? dk[c] : dq[c], 1);
            }
#pragma unroll
            for (int o = 2; o < SL; o <<= 1) {
#pragma unroll
                for (int c = 0; c < NC; ++c) mine[c] += __shfl_xor_sync(0xffffffffu, mine[c], o);
            }
            const float4 par = *reinterpret_cast<const float4*>(sc + COLS);      // beta, decay, k.q
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const float dkt = __shfl_sync(0xffffffffu, mine[c], lane & ~(SL - 1));
                const float u = par.x * (sc[cw + c] - par.y * dkt);
#pragma unroll
                for (int n = 0; n < NR; ++n) S[c][n] = fmaf(kr[n], u, par.y * S[c][n]);
                if (slice == 1 && j + c < V)
                    a.o[(size_t)(s * a.seq_len + t0 + b) * a.ldo + (size_t)h * V + j + c] = fmaf(u, par.z, par.y * mine[c]);
            }
        }
        __syncthreads();                           // the buffer is free for the copies after the next ones
    }
#pragma unroll
    for (int c = 0; c < NC; ++c) {
        if (j + c >= V) continue;
        float* dst = st + (((size_t)((p0 + a.seq_len) & 1) * H + h) * V + j + c) * D;
#pragma unroll
        for (int n = 0; n < NR; ++n) {
            const int i = slice * NR + n;
            if (i < D) dst[i] = S[c][n];
        }
    }
    if (h == 0 && tile == 0) {       // the convolutions' inputs of the last rows go to the ring
        float* ring = st + (size_t)2 * H * D * V;
        const int keep = a.seq_len < a.taps ? a.seq_len : a.taps;
        for (int e = tid; e < keep * C; e += 256) {
            const int b = e / C, c = e - b * C;
            const int i = a.seq_len - keep + b;
            ring[(size_t)((p0 + i) % a.taps) * C + c] = a.proj[(size_t)(s * a.seq_len + i) * a.ldp + a.c_off + c];
        }
    }
}

template <int NR, int SL, int NC>
static int launch_delta_rule(const b200_delta_args* a, cudaStream_t s) {
    constexpr int COLS = NC * 256 / SL;
    const size_t per_token = (size_t)(2 * NR * SL + COLS + 4) * sizeof(float);
    int tb = a->seq_len < kDeltaBatch ? a->seq_len : kDeltaBatch;            // (a decode step stages one token)
    while (tb > 1 && 2 * tb * per_token > 200 * 1024) --tb;                  // (very long rows: fewer tokens per buffer)
    const size_t smem = (size_t)2 * tb * per_token;
    if (smem > 48 * 1024)
        B200_CUDA_CHECK(cudaFuncSetAttribute(delta_rule_kernel<NR, SL, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int qk = a->kv_heads * a->dim;
    const int vec = (a->dim % 4 == 0 && a->ldw % 4 == 0 && qk % 4 == 0 && (reinterpret_cast<uintptr_t>(a->work) & 15) == 0) ? 1 : 0;
    dim3 grid(a->n_seq, a->heads, (a->vdim + COLS - 1) / COLS);
    B200_CUDA_CHECK(launch(delta_rule_kernel<NR, SL, NC>, grid, dim3(256), smem, s, a->pdl != 0, *a, vec, tb));
    return B200_OK;
}

}  // namespace b200

using namespace b200;

static int check_delta(const b200_delta_args* a, const char* who) {
    if (!a || !a->proj || !a->work || (!a->state && !a->state_ptrs)) return fail(B200_EINVAL, "%s: null pointer argument", who);
    if (a->n_seq <= 0 || a->seq_len <= 0 || a->heads <= 0 || a->kv_heads <= 0 || a->heads % a->kv_heads || a->dim <= 0 ||
        a->vdim <= 0 || a->taps <= 0)
        return fail(B200_EINVAL, "%s: bad sizes (heads %d kv_heads %d dim %d vdim %d taps %d)", who, a->heads, a->kv_heads, a->dim,
                    a->vdim, a->taps);
    if (a->n_seq > 1 && a->seq_len > 1 && !a->state_ptrs) return fail(B200_EINVAL, "%s: several sequences need state_ptrs", who);
    return B200_OK;
}

extern "C" int b200_delta_prep(const b200_delta_args* a, void* stream) {
    if (int rc = check_delta(a, "b200_delta_prep")) return rc;
    if (!a->conv_w || !a->A_log || !a->dt_bias) return fail(B200_EINVAL, "b200_delta_prep: parameters missing");
    const size_t smem = (size_t)(2 * a->dim > a->vdim ? 2 * a->dim : a->vdim) * sizeof(float);
    if (smem > 48 * 1024) return fail(B200_ELIMIT, "b200_delta_prep: dim %d exceeds shared memory", a->dim);
    const int rpb = a->seq_len >= 64 ? 8 : 1;
    const dim3 grid(a->n_seq * ((a->seq_len + rpb - 1) / rpb), a->kv_heads + a->heads);
    if (rpb > 1)
        B200_CUDA_CHECK(launch(delta_prep_kernel<32>, grid, dim3(32), smem, static_cast<cudaStream_t>(stream), a->pdl != 0, *a, rpb));
    else
        B200_CUDA_CHECK(launch(delta_prep_kernel<128>, grid, dim3(128), smem, static_cast<cudaStream_t>(stream), a->pdl != 0, *a, rpb));
    return B200_OK;
}

extern "C" int b200_delta_rule(const b200_delta_args* a, void* stream) {
    if (int rc = check_delta(a, "b200_delta_rule")) return rc;
    if (!a->o) return fail(B200_EINVAL, "b200_delta_rule: o missing");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // (few rows per lane: the work of a token is a chain of dependent steps, so the more warps share it the better)
    // a run of tokens: several columns per lane group (shared reads of k and q, independent chains); a decode step:
    // as many blocks as possible, its time is the state's traffic
    const bool run = a->seq_len > 1 && a->vdim >= 32;
    if (a->dim <= 64) return run ? launch_delta_rule<4, 16, 2>(a, s) : launch_delta_rule<4, 16, 1>(a, s);
    if (a->dim <= 128) return run ? launch_delta_rule<4, 32, 2>(a, s) : launch_delta_rule<4, 32, 1>(a, s);
    if (a->dim <= 256) return run ? launch_delta_rule<8, 32, 2>(a, s) : launch_delta_rule<8, 32, 1>(a, s);
    if (a->dim <= 512) return launch_delta_rule<16, 32, 1>(a, s);
    if (a->dim <= 1024) return launch_delta_rule<32, 32, 1>(a, s);
    return fail(B200_ELIMIT, "b200_delta_rule: dim %d > 1024", a->dim);
}
