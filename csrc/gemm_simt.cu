// fp32-accumulating GEMM on the CUDA cores (true 32-bit products): the all-fp32 execution mode of layer-list designs,
// the per-head products around latent attention (batched) and the experts of a mixture (grouped by a device table).
// 64 x 64 output tile, 16-wide k steps, 256 threads with a 4 x 4 micro-tile each.
#include "common.h"
#include "ptx.cuh"

namespace b200 {

constexpr int kTM = 64, kTN = 64, kTK = 16;

__device__ __forceinline__ float ld_any(const void* p, size_t i, int dtype) {
    if (dtype == B200_F32) return static_cast<const float*>(p)[i];
    return h16_to_float(static_cast<const uint16_t*>(p)[i], dtype == B200_BF16);
}

template <bool DUAL>
__global__ void __launch_bounds__(256) gemm_simt_kernel(b200_simt_gemm_args a) {
    __shared__ float As[kTK][kTM + 1];
    __shared__ float Bs[kTK][kTN + 1];
    __shared__ float B2[DUAL ? kTK : 1][kTN + 1];
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int tid = threadIdx.x;
    const int b = blockIdx.z;
    // which rows does this CTA own?
    int r0, rend;
    size_t w_off = (size_t)b * a.w_bs;
    if (a.group_off) {
        int bt = blockIdx.x, g = 0;
        r0 = rend = 0;
        bool found = false;
        for (; g < a.groups; ++g) {
            const int lo = a.group_off[g], hi = a.group_off[g + 1];
            const int tiles = (hi - lo + kTM - 1) / kTM;
            if (bt < tiles) {
                r0 = lo + bt * kTM;
                rend = hi;
                found = true;
                break;
            }
            bt -= tiles;
        }
        if (!found) return;
        w_off += (size_t)g * a.w_gs;
    } else {
        r0 = blockIdx.x * kTM;
        rend = a.T;
        if (r0 >= rend) return;
    }
    const int n0 = blockIdx.y * kTN;
    const char* xb = static_cast<const char*>(a.x);
    const size_t xes = a.x_dtype == B200_F32 ? 4 : 2, wes = a.w_dtype == B200_F32 ? 4 : 2;
    const void* x = xb + (size_t)b * a.x_bs * xes;
    const void* w = static_cast<const char*>(a.w) + w_off * wes;
    const void* w2 = DUAL ? static_cast<const void*>(static_cast<const char*>(a.w2) + w_off * wes) : nullptr;

    // loader mapping: 4 elements per thread per operand: e = tid + i*256 -> (row e/16, k e%16)
    int src_row[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + (tid + i * 256) / kTK;
        src_row[i] = r < rend ? (a.row_src ? a.row_src[r] : r) : -1;
    }
    const int ty = tid / 16, tx = tid % 16;
    float acc[4][4] = {}, acc2[DUAL ? 4 : 1][4] = {};
    for (int k0 = 0; k0 < a.K; k0 += kTK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256, r = e / kTK, k = e % kTK;
            const bool kin = k0 + k < a.K;
            As[k][r] = (kin && src_row[i] >= 0) ? ld_any(x, (size_t)src_row[i] * a.ldx + k0 + k, a.x_dtype) : 0.f;
            const int n = n0 + r;
            const bool nin = kin && n < a.N;
            Bs[k][r] = nin ? ld_any(w, (size_t)n * a.ldw + k0 + k, a.w_dtype) : 0.f;
            if (DUAL) B2[k][r] = nin ? ld_any(w2, (size_t)n * a.ldw + k0 + k, a.w_dtype) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kTK; ++k) {
            float av[4], bv[4], b2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bv[j] = Bs[k][tx * 4 + j];
            if (DUAL) {
#pragma unroll
                for (int j = 0; j < 4; ++j) b2[j] = B2[k][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
                    if (DUAL) acc2[i][j] = fmaf(av[i], b2[j], acc2[i][j]);
                }
        }
        __syncthreads();
    }
    char* ob = static_cast<char*>(a.out);
    const size_t oes = a.out_dtype == B200_F32 ? 4 : 2;
    void* out = ob + (size_t)b * a.o_bs * oes;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + ty * 4 + i;
        if (r >= rend) continue;
        const int dr = a.row_dst ? a.row_dst[r] : r;
        const float sc = a.row_scale ? a.row_scale[r] : 1.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= a.N) continue;
            float v = acc[i][j];
            if (DUAL) v = v / (1.0f + expf(-v)) * acc2[i][j];
            v *= sc;
            if (a.out_dtype == B200_F32)
                static_cast<float*>(out)[(size_t)dr * a.ldo + n] = v;
            else
                static_cast<uint16_t*>(out)[(size_t)dr * a.ldo + n] = float_to_h16(v, a.out_dtype == B200_BF16);
        }
    }
}

// Decode sizes (T <= 16, no grouping): one warp per output feature, the weight row streamed once with coalesced loads
// and reused for every token - the tile kernel would leave all but a few CTAs idle and spend its time in barriers.
constexpr int kRowsMax = 16;
__global__ void __launch_bounds__(256) gemm_rows_kernel(b200_simt_gemm_args a) {
    pdl_wait_prior_grid();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, n = blockIdx.x * 8 + (threadIdx.x >> 5), b = blockIdx.y;
    if (n >= a.N) return;
    const size_t xes = a.x_dtype == B200_F32 ? 4 : 2, wes = a.w_dtype == B200_F32 ? 4 : 2;
    const void* x = static_cast<const char*>(a.x) + (size_t)b * a.x_bs * xes;
    const void* w = static_cast<const char*>(a.w) + ((size_t)b * a.w_bs + (size_t)n * a.ldw) * wes;
    float acc[kRowsMax];
#pragma unroll
    for (int t = 0; t < kRowsMax; ++t) acc[t] = 0.f;
#pragma unroll 4
    for (int k = lane; k < a.K; k += 32) {
        const float wv = ld_any(w, k, a.w_dtype);
#pragma unroll
        for (int t = 0; t < kRowsMax; ++t)
            if (t < a.T) acc[t] = fmaf(ld_any(x, (size_t)t * a.ldx + k, a.x_dtype), wv, acc[t]);
    }
    char* ob = static_cast<char*>(a.out) + (size_t)b * a.o_bs * (a.out_dtype == B200_F32 ? 4 : 2);
#pragma unroll
    for (int t = 0; t < kRowsMax; ++t) {
        if (t >= a.T) break;
        float v = acc[t];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) {
            if (a.out_dtype == B200_F32)
                reinterpret_cast<float*>(ob)[(size_t)t * a.ldo + n] = v;
            else
                reinterpret_cast<uint16_t*>(ob)[(size_t)t * a.ldo + n] = float_to_h16(v, a.out_dtype == B200_BF16);
        }
    }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_gemm_simt(const b200_simt_gemm_args* a, void* stream) {
    if (!a || !a->x || !a->w || !a->out) return fail(B200_EINVAL, "b200_gemm_simt: null pointer argument");
    if (a->T <= 0 || a->N <= 0 || a->K <= 0) return fail(B200_EINVAL, "b200_gemm_simt: bad sizes T=%d N=%d K=%d", a->T, a->N, a->K);
    if (a->group_off && a->groups <= 0) return fail(B200_EINVAL, "b200_gemm_simt: group table without groups");
    const int batch = a->batch > 0 ? a->batch : 1;
    int row_tiles = (a->T + kTM - 1) / kTM;
    if (a->group_off) row_tiles += a->groups;      // every group may end in a partial tile
    dim3 grid(row_tiles, (a->N + kTN - 1) / kTN, batch);
    if (grid.y > 65535 || grid.z > 65535) return fail(B200_ELIMIT, "b200_gemm_simt: grid too large");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (a->T <= kRowsMax && !a->group_off && !a->w2 && !a->row_src && !a->row_dst && !a->row_scale && batch <= 65535) {
        B200_CUDA_CHECK(launch(gemm_rows_kernel, dim3((a->N + 7) / 8, batch), dim3(256), 0, s, a->pdl != 0, *a));
        return B200_OK;
    }
    if (a->w2)
        B200_CUDA_CHECK(launch(gemm_simt_kernel<true>, grid, dim3(256), 0, s, a->pdl != 0, *a));
    else
        B200_CUDA_CHECK(launch(gemm_simt_kernel<false>, grid, dim3(256), 0, s, a->pdl != 0, *a));
    return B200_OK;
}
