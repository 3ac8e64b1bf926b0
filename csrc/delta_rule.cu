// Gated delta rule behind short causal convolutions: a matrix state per head that decays, is corrected towards the
// current value along the current key and is read with the query.  Everything here is fp32.
//   prep  (one block per row):   convolutions + silu, unit-length q / k, beta and decay of every head
//   rule  (sequential in time):  S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
// A sequence's state lives with its cache: two copies of the heads' matrices (a launch whose first token is at position
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
__global__ void __launch_bounds__(256) delta_prep_kernel(b200_delta_args a) {
    extern __shared__ float y[];                   // [channels] convolved + activated
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int r = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int s = r / a.seq_len, i = r - s * a.seq_len;
    const int p = (a.pos ? a.pos[s] : a.pos0) + i;
    const int qk = a.kv_heads * a.dim, C = 2 * qk + a.heads * a.vdim, taps = a.taps;
    const float* ring = delta_state(a, s) + (size_t)2 * a.heads * a.dim * a.vdim;
    const float* row = a.proj + (size_t)r * a.ldp + a.c_off;
    for (int c = tid; c < C; c += 256) {
        const float* w = a.conv_w + (size_t)c * taps;
        float acc = 0.f;
        for (int b = taps - 1; b >= 0; --b) {      // oldest input first
            if (p - b < 0) continue;               // before the sequence's start: zero
            const float x = b <= i ? row[c - (ptrdiff_t)b * a.ldp] : ring[(size_t)((p - b) % taps) * C + c];
            acc = fmaf(w[taps - 1 - b], x, acc);
        }
        y[c] = acc / (1.0f + expf(-acc));
    }
    __syncthreads();
    float* out = a.work + (size_t)r * a.ldw;
    const float qscale = rsqrtf((float)a.dim);
    for (int hh = warp; hh < 2 * a.kv_heads; hh += 8) {      // q heads, then k heads
        const float* src = y + hh * a.dim;
        float ss = 0.f;
        for (int d = lane; d < a.dim; d += 32) ss = fmaf(src[d], src[d], ss);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float f = (1.0f / sqrtf(ss + a.unit_eps)) * (hh < a.kv_heads ? qscale : 1.0f);
        for (int d = lane; d < a.dim; d += 32) out[hh * a.dim + d] = src[d] * f;
    }
    for (int c = 2 * qk + tid; c < C; c += 256) out[c] = y[c];
    for (int h = tid; h < a.heads; h += 256) {
        const float* rr = a.proj + (size_t)r * a.ldp;
        out[C + h] = 1.0f / (1.0f + expf(-rr[a.b_off + h]));
        out[C + a.heads + h] = expf(-expf(a.A_log[h]) * softplus32(rr[a.a_off + h] + a.dt_bias[h]));
    }
}

// ------------------------------------------------------------------ rule
constexpr int kDeltaCols = 64;       // columns of S per block (8 per warp)
constexpr int kDeltaBatch = 16;      // tokens staged in shared memory at a time

// Block = (sequence, head, 64 columns of S).  Lane = slice * 8 + column: column j's rows i = slice + 4 n are in the
// registers of 4 lanes, dot products meet by two shuffles.
template <int NR>
__global__ void __launch_bounds__(256) delta_rule_kernel(b200_delta_args a) {
    extern __shared__ float sm[];    // per staged token: k [dim] | q [dim] | v [64] | beta, decay
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int s = blockIdx.x, h = blockIdx.y, tile = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int slice = lane >> 3, j = tile * kDeltaCols + warp * 8 + (lane & 7);
    const int D = a.dim, V = a.vdim, H = a.heads;
    const int g = h / (H / a.kv_heads);
    const int qk = a.kv_heads * D, C = 2 * qk + H * V;
    const int p0 = a.pos ? a.pos[s] : a.pos0;
    const bool col = j < V;
    float* st = delta_state(a, s);
    float S[NR];
    {
        const float* src = st + ((size_t)(p0 & 1) * H + h) * D * V;
#pragma unroll
        for (int n = 0; n < NR; ++n) {
            const int i = slice + 4 * n;
            S[n] = (p0 > 0 && col && i < D) ? src[(size_t)i * V + j] : 0.f;
        }
    }
    const int stride = 2 * D + kDeltaCols + 2;
    for (int t0 = 0; t0 < a.seq_len; t0 += kDeltaBatch) {
        const int nb = a.seq_len - t0 < kDeltaBatch ? a.seq_len - t0 : kDeltaBatch;
        __syncthreads();
        for (int e = tid; e < nb * stride; e += 256) {
            const int b = e / stride, c = e - b * stride;
            const float* w = a.work + (size_t)(s * a.seq_len + t0 + b) * a.ldw;
            float v;
            if (c < D)
                v = w[qk + g * D + c];                        // key
            else if (c < 2 * D)
                v = w[g * D + (c - D)];                       // query
            else if (c < 2 * D + kDeltaCols) {
                const int jj = tile * kDeltaCols + (c - 2 * D);
                v = jj < V ? w[2 * qk + h * V + jj] : 0.f;    // value columns of this block
            } else
                v = w[C + (c - 2 * D - kDeltaCols) * H + h];  // beta, decay
            sm[e] = v;
        }
        __syncthreads();
        for (int b = 0; b < nb; ++b) {
            const float* kk = sm + b * stride;
            const float* qq = kk + D;
            const float vj = kk[2 * D + warp * 8 + (lane & 7)];
            const float beta = kk[2 * D + kDeltaCols], dec = kk[2 * D + kDeltaCols + 1];
            float dk = 0.f, dq = 0.f, kq = 0.f;
#pragma unroll
            for (int n = 0; n < NR; ++n) {
                const int i = slice + 4 * n;
                const float ki = i < D ? kk[i] : 0.f, qi = i < D ? qq[i] : 0.f;
                dk = fmaf(S[n], ki, dk);
                dq = fmaf(S[n], qi, dq);
                kq = fmaf(ki, qi, kq);
            }
            dk += __shfl_xor_sync(0xffffffffu, dk, 8);
            dq += __shfl_xor_sync(0xffffffffu, dq, 8);
            kq += __shfl_xor_sync(0xffffffffu, kq, 8);
            dk += __shfl_xor_sync(0xffffffffu, dk, 16);
            dq += __shfl_xor_sync(0xffffffffu, dq, 16);
            kq += __shfl_xor_sync(0xffffffffu, kq, 16);
            const float u = beta * (vj - dec * dk);
#pragma unroll
            for (int n = 0; n < NR; ++n) {
                const int i = slice + 4 * n;
                S[n] = fmaf(i < D ? kk[i] : 0.f, u, dec * S[n]);
            }
            if (slice == 0 && col) a.o[(size_t)(s * a.seq_len + t0 + b) * a.ldo + (size_t)h * V + j] = fmaf(u, kq, dec * dq);
        }
    }
    {
        float* dst = st + ((size_t)((p0 + a.seq_len) & 1) * H + h) * D * V;
#pragma unroll
        for (int n = 0; n < NR; ++n) {
            const int i = slice + 4 * n;
            if (col && i < D) dst[(size_t)i * V + j] = S[n];
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

template <int NR>
static int launch_delta_rule(const b200_delta_args* a, cudaStream_t s) {
    const size_t smem = (size_t)kDeltaBatch * (2 * a->dim + kDeltaCols + 2) * sizeof(float);
    dim3 grid(a->n_seq, a->heads, (a->vdim + kDeltaCols - 1) / kDeltaCols);
    B200_CUDA_CHECK(launch(delta_rule_kernel<NR>, grid, dim3(256), smem, s, a->pdl != 0, *a));
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
    const size_t smem = (size_t)(2 * a->kv_heads * a->dim + a->heads * a->vdim) * sizeof(float);
    if (smem > 200 * 1024) return fail(B200_ELIMIT, "b200_delta_prep: %zu B of channels exceed shared memory", smem);
    if (smem > 48 * 1024)
        B200_CUDA_CHECK(cudaFuncSetAttribute(delta_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    B200_CUDA_CHECK(launch(delta_prep_kernel, dim3(a->n_seq * a->seq_len), dim3(256), smem, static_cast<cudaStream_t>(stream),
                           a->pdl != 0, *a));
    return B200_OK;
}

extern "C" int b200_delta_rule(const b200_delta_args* a, void* stream) {
    if (int rc = check_delta(a, "b200_delta_rule")) return rc;
    if (!a->o) return fail(B200_EINVAL, "b200_delta_rule: o missing");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int nr = (a->dim + 3) / 4;
    if (nr <= 8) return launch_delta_rule<8>(a, s);
    if (nr <= 16) return launch_delta_rule<16>(a, s);
    if (nr <= 32) return launch_delta_rule<32>(a, s);
    if (nr <= 64) return launch_delta_rule<64>(a, s);
    return fail(B200_ELIMIT, "b200_delta_rule: dim %d > 256", a->dim);
}
