// Softmax attention with a sink for prompt-size chunks of one session on the tensor cores (16-bit caches).
// Flash attention over the session's key / value planes (all heads of a position side by side in one row):
//   S = q . k^T                 mma.sync m16n8k16, 16-bit in, fp32 out (the score scale is already folded into q)
//   online softmax in fp32 registers whose running state starts at (m = 0, l = sink): the sink is one more key of
//   score 0 without a value
//   O += P . V with P split into two 16-bit terms (hi + lo), so the weights enter the product with ~16 bits
//   out = O / l * sigmoid(gate logit of the head)
// One block = 64 consecutive queries of one head (4 warps x 16 rows), keys in tiles of 64 up to the block's last
// query; the next tile is fetched by cp.async into a second shared-memory buffer under the current one's math.
// Blocks with the most keys are launched first.
#include "common.h"
#include "mma.cuh"
#include "ptx.cuh"

namespace b200 {

constexpr int kSinkQT = 64, kSinkKT = 64;

struct SinkMmaParams {
    b200_sink_attn_args a;
    const uint16_t* kc;
    const uint16_t* vc;
    int is_bf16, vec;
};

// NV = value n-tiles of 8 columns (vdim <= 8 * NV)
template <int NV>
__global__ void __launch_bounds__(128) sink_attn_mma_kernel(SinkMmaParams p) {
    extern __shared__ __align__(16) uint16_t smem16[];
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const b200_sink_attn_args& a = p.a;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
    const int h = blockIdx.y, q0 = (gridDim.x - 1 - blockIdx.x) * kSinkQT;
    const int kvh = h / (a.heads / a.kv_heads);
    const int dq = a.dim, dqp = (dq + 15) / 16 * 16, ldq = dqp + 8;              // +8 halves: rows land on different banks
    const int ldv = NV * 8 + 8;
    uint16_t* Qs = smem16;                       // [64][ldq]
    uint16_t* Kb = Qs + kSinkQT * ldq;           // 2 x [64][ldq]
    uint16_t* Vb = Kb + 2 * kSinkKT * ldq;       // 2 x [64][ldv]   (key major; transposed by ldmatrix on the way out)
    const int bf = p.is_bf16;
    const bool vec = p.vec != 0;
    for (int e = tid; e < kSinkQT * dqp; e += 128) {
        const int r = e / dqp, d = e - r * dqp;
        float v = 0.f;
        if (q0 + r < a.T && d < dq) v = a.proj[(size_t)(q0 + r) * a.ldp + a.q_off + h * dq + d];
        Qs[r * ldq + d] = float_to_h16(v, bf);
    }
    const int P0 = a.pos0 + q0;
    const int plast = a.pos0 + (q0 + kSinkQT < a.T ? q0 + kSinkQT : a.T) - 1;
    float o[NV][4];
#pragma unroll
    for (int i = 0; i < NV; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    const bool sink = a.sink > 0.f;
    float m0 = sink ? 0.f : -INFINITY, m1 = m0, l0 = sink ? a.sink : 0.f, l1 = l0;   // rows g and g + 8 of this warp's 16
    const int qp0 = P0 + warp * 16 + g, qp1 = qp0 + 8;
    const size_t re = (size_t)a.row_elems;
    auto load_tile = [&](int buf, int k0) {
        uint16_t* Ks = Kb + buf * kSinkKT * ldq;
        uint16_t* Vs = Vb + buf * kSinkKT * ldv;
        if (vec) {
            const int cpr = dqp / 8;
            for (int e = tid; e < kSinkKT * cpr; e += 128) {
                const int j = e / cpr, d = (e - j * cpr) * 8;
                const int kp = k0 + j;
                const bool in = kp <= plast && d < dq;
                cp_async16(Ks + j * ldq + d, in ? p.kc + (size_t)kp * re + kvh * dq + d : p.kc, in ? 16 : 0);
            }
            for (int e = tid; e < kSinkKT * NV; e += 128) {
                const int j = e / NV, c = (e - j * NV) * 8;
                const int kp = k0 + j;
                const bool in = kp <= plast && c < a.vdim;
                cp_async16(Vs + j * ldv + c, in ? p.vc + (size_t)kp * re + kvh * a.vdim + c : p.vc, in ? 16 : 0);
            }
        } else {
            for (int e = tid; e < kSinkKT * dqp; e += 128) {
                const int j = e / dqp, d = e - j * dqp;
                const int kp = k0 + j;
                Ks[j * ldq + d] = (kp <= plast && d < dq) ? p.kc[(size_t)kp * re + kvh * dq + d] : (uint16_t)0;
            }
            for (int e = tid; e < kSinkKT * NV * 8; e += 128) {
                const int j = e / (NV * 8), c = e - j * (NV * 8);
                const int kp = k0 + j;
                Vs[j * ldv + c] = (kp <= plast && c < a.vdim) ? p.vc[(size_t)kp * re + kvh * a.vdim + c] : (uint16_t)0;
            }
        }
        cp_async_commit();
    };
    load_tile(0, 0);
    int buf = 0;
    for (int k0 = 0; k0 <= plast; k0 += kSinkKT, buf ^= 1) {
        if (k0 + kSinkKT <= plast) {
            load_tile(buf ^ 1, k0 + kSinkKT);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint16_t* Ks = Kb + buf * kSinkKT * ldq;
        const uint16_t* Vs = Vb + buf * kSinkKT * ldv;
        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
        const uint16_t* qrow0 = Qs + (warp * 16 + g) * ldq;
        const uint16_t* qrow1 = qrow0 + 8 * ldq;
        for (int kk = 0; kk < dqp; kk += 16) {
            uint32_t af[4];
            af[0] = *reinterpret_cast<const uint32_t*>(qrow0 + kk + 2 * tq);
            af[1] = *reinterpret_cast<const uint32_t*>(qrow1 + kk + 2 * tq);
            af[2] = *reinterpret_cast<const uint32_t*>(qrow0 + kk + 8 + 2 * tq);
            af[3] = *reinterpret_cast<const uint32_t*>(qrow1 + kk + 8 + 2 * tq);
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const uint16_t* krow = Ks + (n * 8 + g) * ldq + kk + 2 * tq;
                mma_16816(s[n], af, *reinterpret_cast<const uint32_t*>(krow), *reinterpret_cast<const uint32_t*>(krow + 8), bf);
            }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int kp = k0 + n * 8 + 2 * tq + c;
                if (kp > qp0) s[n][c] = -INFINITY;
                if (kp > qp1) s[n][2 + c] = -INFINITY;
                mx0 = fmaxf(mx0, s[n][c]);
                mx1 = fmaxf(mx1, s[n][2 + c]);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        // (a row may have seen no key yet: keep everything at zero then, exp(-inf - -inf) must not be evaluated)
        const float al0 = mn0 == -INFINITY ? 1.f : expf(m0 - mn0), al1 = mn1 == -INFINITY ? 1.f : expf(m1 - mn1);
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                s[n][c] = mn0 == -INFINITY ? 0.f : expf(s[n][c] - mn0);
                s[n][2 + c] = mn1 == -INFINITY ? 0.f : expf(s[n][2 + c] - mn1);
                ps0 += s[n][c];
                ps1 += s[n][2 + c];
            }
        }
        ps0 += __shfl_xor_sync(0xffffffffu, ps0, 1);
        ps0 += __shfl_xor_sync(0xffffffffu, ps0, 2);
        ps1 += __shfl_xor_sync(0xffffffffu, ps1, 1);
        ps1 += __shfl_xor_sync(0xffffffffu, ps1, 2);
        l0 = l0 * al0 + ps0;
        l1 = l1 * al1 + ps1;
        m0 = mn0;
        m1 = mn1;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            o[i][0] *= al0;
            o[i][1] *= al0;
            o[i][2] *= al1;
            o[i][3] *= al1;
        }
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {                                         // 16 keys per step = two score n-tiles
            uint32_t ah[4], alo[4];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const float* sv = s[2 * ks + half];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const float x0 = sv[2 * r], x1 = sv[2 * r + 1];
                    const uint16_t h0 = float_to_h16(x0, bf), h1 = float_to_h16(x1, bf);
                    ah[half * 2 + r] = (uint32_t)h0 | ((uint32_t)h1 << 16);
                    alo[half * 2 + r] = pack2(x0 - h16_to_float(h0, bf), x1 - h16_to_float(h1, bf), bf);
                }
            }
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                uint32_t b0, b1;
                ldmatrix_x2_trans(b0, b1, Vs + (ks * 16 + (lane & 15)) * ldv + i * 8);
                mma_16816(o[i], ah, b0, b1, bf);
                mma_16816(o[i], alo, b0, b1, bf);
            }
        }
        __syncthreads();
    }
    const int r0 = q0 + warp * 16 + g, r1 = r0 + 8;
    float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
    if (r0 < a.T) i0 *= 1.0f / (1.0f + expf(-a.proj[(size_t)r0 * a.ldp + a.g_off + h]));
    if (r1 < a.T) i1 *= 1.0f / (1.0f + expf(-a.proj[(size_t)r1 * a.ldp + a.g_off + h]));
    uint16_t* out = static_cast<uint16_t*>(a.out);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int col = i * 8 + 2 * tq + c;
            if (col >= a.vdim) continue;
            if (r0 < a.T) out[(size_t)r0 * a.ldo + h * a.vdim + col] = float_to_h16(o[i][c] * i0, bf);
            if (r1 < a.T) out[(size_t)r1 * a.ldo + h * a.vdim + col] = float_to_h16(o[i][2 + c] * i1, bf);
        }
    }
}

template <int NV>
static int launch_sink_mma(const SinkMmaParams& p, size_t smem, cudaStream_t s) {
    if (smem > 48 * 1024)
        B200_CUDA_CHECK(cudaFuncSetAttribute(sink_attn_mma_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    B200_CUDA_CHECK(launch(sink_attn_mma_kernel<NV>, dim3((p.a.T + kSinkQT - 1) / kSinkQT, p.a.heads), dim3(128), smem, s,
                           p.a.pdl != 0, p));
    return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_sink_attn_prefill(const b200_sink_attn_args* a, void* stream) {
    if (!a || !a->proj || !a->k_cache || !a->v_cache || !a->out) return fail(B200_EINVAL, "b200_sink_attn_prefill: null pointer argument");
    if (a->kv_ptrs || a->pos) return fail(B200_EINVAL, "b200_sink_attn_prefill: one session with consecutive positions only");
    if (a->T <= 0 || a->heads <= 0 || a->kv_heads <= 0 || a->heads % a->kv_heads || a->dim <= 0 || a->vdim <= 0 || a->pos0 < 0 ||
        a->row_elems < a->kv_heads * a->dim || a->row_elems < a->kv_heads * a->vdim)
        return fail(B200_EINVAL, "b200_sink_attn_prefill: bad sizes");
    if ((a->cache_dtype != B200_F16 && a->cache_dtype != B200_BF16) || a->out_dtype != a->cache_dtype)
        return fail(B200_EINVAL, "b200_sink_attn_prefill: 16-bit cache and output of one type");
    if (a->vdim > 256) return fail(B200_ELIMIT, "b200_sink_attn_prefill: vdim %d > 256", a->vdim);
    SinkMmaParams p;
    p.a = *a;
    p.kc = static_cast<const uint16_t*>(a->k_cache);
    p.vc = static_cast<const uint16_t*>(a->v_cache);
    p.is_bf16 = a->cache_dtype == B200_BF16 ? 1 : 0;
    p.vec = (a->dim % 8 == 0 && a->vdim % 8 == 0 && a->row_elems % 8 == 0 && (reinterpret_cast<uintptr_t>(a->k_cache) & 15) == 0 &&
             (reinterpret_cast<uintptr_t>(a->v_cache) & 15) == 0) ? 1 : 0;
    const int dqp = (a->dim + 15) / 16 * 16;
    const int nv = (a->vdim + 7) / 8;
    const int NV = nv <= 4 ? 4 : nv <= 8 ? 8 : nv <= 16 ? 16 : 32;
    const size_t smem = ((size_t)(kSinkQT + 2 * kSinkKT) * (dqp + 8) + (size_t)2 * kSinkKT * (NV * 8 + 8)) * sizeof(uint16_t);
    if (smem > 200 * 1024) return fail(B200_ELIMIT, "b200_sink_attn_prefill: dim %d exceeds shared memory", a->dim);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (NV) {
        case 4: return launch_sink_mma<4>(p, smem, s);
        case 8: return launch_sink_mma<8>(p, smem, s);
        case 16: return launch_sink_mma<16>(p, smem, s);
        default: return launch_sink_mma<32>(p, smem, s);
    }
}
