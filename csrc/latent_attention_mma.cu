// Latent attention for prompt-size inputs on the tensor cores (16-bit modes).
// The latents of the rows a chunk can see are expanded once per layer by a tensor-core GEMM into per-head keys and
// values (kvx = cache rows . [W_uk | W_uv]^T); this kernel is then a sliding-window flash attention over them:
//   S = [q_unrotated | q_rotated] . [k_unrotated(head) | k_rotated(shared)]^T   mma.sync m16n8k16, 16-bit in, fp32 out
//   online softmax in fp32 registers
//   O += P . V with P split into two 16-bit terms (hi + lo), so the weights enter the product with ~16 bits
// One block = 64 consecutive queries of one head (4 warps x 16 rows), keys in tiles of 64; the next key / value tile is
// fetched by cp.async into a second shared-memory buffer while the tensor cores work on the current one.
#include "common.h"
#include "mma.cuh"
#include "ptx.cuh"

namespace b200 {

struct LatentMmaParams {
    const float* proj;        // [T, ldp] fp32: q at q_off, head stride dim + rot (rotated part already rotated)
    const uint16_t* kvx;      // [rows, ldkv]: k_unrotated at h * dim, v at v_off + h * vdim; row r = key position s0 + r
    const uint16_t* cache;    // session rows [.., row_elems]: rotated key part at column kv_rank
    uint16_t* out;            // [T, ldo]: head h at h * vdim
    int ldp, q_off, ldkv, v_off, row_elems, kv_rank, ldo;
    int T, heads, dim, rot, vdim, pos0, s0, window;
    float scale;
    int is_bf16;
    int vec;                  // sizes and addresses allow 16-byte tile loads
};

constexpr int kQT = 64, kKT = 64;

// NV = value n-tiles of 8 columns (vdim <= 8 * NV)
template <int NV>
__global__ void __launch_bounds__(128) latent_attn_mma_kernel(LatentMmaParams p) {
    extern __shared__ __align__(16) uint16_t smem16[];
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
    const int h = blockIdx.y, q0 = blockIdx.x * kQT;
    const int dq = p.dim + p.rot, dqp = (dq + 15) / 16 * 16, ldq = dqp + 8;      // +8 halves: rows land on different banks
    const int ldv = NV * 8 + 8;
    uint16_t* Qs = smem16;                       // [64][ldq]
    uint16_t* Kb = Qs + kQT * ldq;               // 2 x [64][ldq]
    uint16_t* Vb = Kb + 2 * kKT * ldq;           // 2 x [64][ldv]   (key major; transposed by ldmatrix on the way out)
    const int bf = p.is_bf16;
    const bool vec = p.vec != 0;
    // ---- Q tile: fp32 -> 16-bit, zero beyond T and beyond dq
    for (int e = tid; e < kQT * dqp; e += 128) {
        const int r = e / dqp, d = e - r * dqp;
        float v = 0.f;
        if (q0 + r < p.T && d < dq) v = p.proj[(size_t)(q0 + r) * p.ldp + p.q_off + h * dq + d];
        Qs[r * ldq + d] = float_to_h16(v, bf);
    }
    const int P0 = p.pos0 + q0;                                                  // position of the tile's first query
    const int plast = p.pos0 + (q0 + kQT < p.T ? q0 + kQT : p.T) - 1;            // ... and of its last one
    int kmin = P0 - p.window + 1;
    if (kmin < 0) kmin = 0;
    float o[NV][4];
#pragma unroll
    for (int i = 0; i < NV; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;                    // rows g and g + 8 of this warp's 16
    const int qp0 = P0 + warp * 16 + g, qp1 = qp0 + 8;
    auto load_tile = [&](int buf, int k0) {
        uint16_t* Ks = Kb + buf * kKT * ldq;
        uint16_t* Vs = Vb + buf * kKT * ldv;
        if (vec) {       // every 8-element group lies in one source and is 16-byte aligned there
            const int cpr = dqp / 8;
            for (int e = tid; e < kKT * cpr; e += 128) {
                const int j = e / cpr, d = (e - j * cpr) * 8;
                const int kp = k0 + j;
                const uint16_t* src = p.kvx;
                int bytes = 0;
                if (kp <= plast) {
                    if (d < p.dim) {
                        src = p.kvx + (size_t)(kp - p.s0) * p.ldkv + h * p.dim + d;
                        bytes = 16;
                    } else if (d < dq) {
                        src = p.cache + (size_t)kp * p.row_elems + p.kv_rank + (d - p.dim);
                        bytes = 16;
                    }
                }
                cp_async16(Ks + j * ldq + d, src, bytes);
            }
            for (int e = tid; e < kKT * NV; e += 128) {
                const int j = e / NV, c = (e - j * NV) * 8;
                const int kp = k0 + j;
                const bool in = kp <= plast && c < p.vdim;
                const uint16_t* src = in ? p.kvx + (size_t)(kp - p.s0) * p.ldkv + p.v_off + h * p.vdim + c : p.kvx;
                cp_async16(Vs + j * ldv + c, src, in ? 16 : 0);
            }
        } else {
            for (int e = tid; e < kKT * dqp; e += 128) {
                const int j = e / dqp, d = e - j * dqp;
                const int kp = k0 + j;
                uint16_t v = 0;
                if (kp <= plast) {
                    if (d < p.dim)
                        v = p.kvx[(size_t)(kp - p.s0) * p.ldkv + h * p.dim + d];
                    else if (d < dq)
                        v = p.cache[(size_t)kp * p.row_elems + p.kv_rank + (d - p.dim)];
                }
                Ks[j * ldq + d] = v;
            }
            for (int e = tid; e < kKT * NV * 8; e += 128) {
                const int j = e / (NV * 8), c = e - j * (NV * 8);
                const int kp = k0 + j;
                uint16_t v = 0;
                if (kp <= plast && c < p.vdim) v = p.kvx[(size_t)(kp - p.s0) * p.ldkv + p.v_off + h * p.vdim + c];
                Vs[j * ldv + c] = v;
            }
        }
        cp_async_commit();
    };
    load_tile(0, kmin);
    int buf = 0;
    for (int k0 = kmin; k0 <= plast; k0 += kKT, buf ^= 1) {
        if (k0 + kKT <= plast) {                                                 // fetch the next tile under this one's math
            load_tile(buf ^ 1, k0 + kKT);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();                                                         // tile `buf` (and Q) visible to all warps
        const uint16_t* Ks = Kb + buf * kKT * ldq;
        const uint16_t* Vs = Vb + buf * kKT * ldv;
        // ---- S = Q K^T for this warp's 16 rows
        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
        const uint16_t* qrow0 = Qs + (warp * 16 + g) * ldq;
        const uint16_t* qrow1 = qrow0 + 8 * ldq;
        for (int kk = 0; kk < dqp; kk += 16) {
            uint32_t a[4];
            a[0] = *reinterpret_cast<const uint32_t*>(qrow0 + kk + 2 * tq);
            a[1] = *reinterpret_cast<const uint32_t*>(qrow1 + kk + 2 * tq);
            a[2] = *reinterpret_cast<const uint32_t*>(qrow0 + kk + 8 + 2 * tq);
            a[3] = *reinterpret_cast<const uint32_t*>(qrow1 + kk + 8 + 2 * tq);
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const uint16_t* krow = Ks + (n * 8 + g) * ldq + kk + 2 * tq;
                mma_16816(s[n], a, *reinterpret_cast<const uint32_t*>(krow), *reinterpret_cast<const uint32_t*>(krow + 8), bf);
            }
        }
        // ---- mask, online softmax (fp32)
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int kp = k0 + n * 8 + 2 * tq + c;
                const bool ok0 = kp <= qp0 && qp0 - kp < p.window && kp <= plast;
                const bool ok1 = kp <= qp1 && qp1 - kp < p.window && kp <= plast;
                s[n][c] = ok0 ? s[n][c] * p.scale : -INFINITY;
                s[n][2 + c] = ok1 ? s[n][2 + c] * p.scale : -INFINITY;
                mx0 = fmaxf(mx0, s[n][c]);
                mx1 = fmaxf(mx1, s[n][2 + c]);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        // (a row may see no key of this tile: keep everything at zero then, exp(-inf - -inf) must not be evaluated)
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
        // ---- O += P V, P as hi + lo 16-bit terms
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {                                         // 16 keys per step = two score n-tiles
            uint32_t ah[4], alo[4];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const float* sv = s[2 * ks + half];
#pragma unroll
                for (int r = 0; r < 2; ++r) {                                    // r = 0: row g, r = 1: row g + 8
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
        __syncthreads();                                                         // all warps are done with tile `buf`
    }
    // ---- normalise and store (16-bit)
    const int r0 = q0 + warp * 16 + g, r1 = r0 + 8;
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int col = i * 8 + 2 * tq + c;
            if (col >= p.vdim) continue;
            if (r0 < p.T) p.out[(size_t)r0 * p.ldo + h * p.vdim + col] = float_to_h16(o[i][c] * i0, bf);
            if (r1 < p.T) p.out[(size_t)r1 * p.ldo + h * p.vdim + col] = float_to_h16(o[i][2 + c] * i1, bf);
        }
    }
}

template <int NV>
static int launch_mma(const LatentMmaParams& p, size_t smem, cudaStream_t s, bool pdl) {
    if (smem > 48 * 1024)
        B200_CUDA_CHECK(cudaFuncSetAttribute(latent_attn_mma_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    B200_CUDA_CHECK(launch(latent_attn_mma_kernel<NV>, dim3((p.T + kQT - 1) / kQT, p.heads), dim3(128), smem, s, pdl, p));
    return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_latent_attn_prefill(const float* proj, int32_t ldp, int32_t q_off, const void* kvx, int32_t ldkv,
                                        int32_t v_off, const void* cache, int32_t row_elems, int32_t kv_rank, void* out,
                                        int32_t ldo, int32_t T, int32_t heads, int32_t dim, int32_t rot, int32_t vdim,
                                        int32_t pos0, int32_t s0, int32_t window, float scale, int32_t dtype, int32_t pdl,
                                        void* stream) {
    if (!proj || !kvx || !cache || !out) return fail(B200_EINVAL, "b200_latent_attn_prefill: null pointer argument");
    if (T <= 0 || heads <= 0 || dim < 0 || rot < 0 || dim + rot <= 0 || vdim <= 0 || window <= 0 || s0 < 0 || s0 > pos0 ||
        (dtype != B200_F16 && dtype != B200_BF16))
        return fail(B200_EINVAL, "b200_latent_attn_prefill: bad argument");
    if (pos0 - window + 1 < s0 && s0 > 0) return fail(B200_EINVAL, "b200_latent_attn_prefill: kvx starts behind the first visible key");
    if (vdim > 256) return fail(B200_ELIMIT, "b200_latent_attn_prefill: vdim %d > 256", vdim);
    LatentMmaParams p;
    p.proj = proj; p.kvx = static_cast<const uint16_t*>(kvx); p.cache = static_cast<const uint16_t*>(cache);
    p.out = static_cast<uint16_t*>(out);
    p.ldp = ldp; p.q_off = q_off; p.ldkv = ldkv; p.v_off = v_off; p.row_elems = row_elems; p.kv_rank = kv_rank; p.ldo = ldo;
    p.T = T; p.heads = heads; p.dim = dim; p.rot = rot; p.vdim = vdim; p.pos0 = pos0; p.s0 = s0; p.window = window;
    p.scale = scale; p.is_bf16 = dtype == B200_BF16 ? 1 : 0;
    p.vec = (dim % 8 == 0 && rot % 8 == 0 && vdim % 8 == 0 && ldkv % 8 == 0 && v_off % 8 == 0 && row_elems % 8 == 0 &&
             kv_rank % 8 == 0 && (reinterpret_cast<uintptr_t>(kvx) & 15) == 0 && (reinterpret_cast<uintptr_t>(cache) & 15) == 0)
                ? 1 : 0;
    const int dqp = (dim + rot + 15) / 16 * 16;
    const int nv = (vdim + 7) / 8;
    const int NV = nv <= 4 ? 4 : nv <= 8 ? 8 : nv <= 16 ? 16 : 32;
    const size_t smem = ((size_t)(kQT + 2 * kKT) * (dqp + 8) + (size_t)2 * kKT * (NV * 8 + 8)) * sizeof(uint16_t);
    if (smem > 200 * 1024) return fail(B200_ELIMIT, "b200_latent_attn_prefill: dim + rot = %d exceeds shared memory", dim + rot);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (NV) {
        case 4: return launch_mma<4>(p, smem, s, pdl != 0);
        case 8: return launch_mma<8>(p, smem, s, pdl != 0);
        case 16: return launch_mma<16>(p, smem, s, pdl != 0);
        default: return launch_mma<32>(p, smem, s, pdl != 0);
    }
}
