// Per-head matrix products on tensor cores, all bfloat16 with fp32 accumulation:
//
//   Y[t][h*y_head + n] = sum_k W[h][n][k] * X[t][h*x_head + k]      for every head h
//
// X and Y are rows of tokens in which head h's block starts h*x_head (h*y_head) entries into the row;
// W is [heads][N][K], contiguous.  This is the small batched product in front of and behind an attention
// over a shared low-rank row per token: the plain query channels carried into the row's space (K = head
// channels, N = rank) and the weighted rows carried out to each head's values (K = rank, N = value
// channels).  A CTA owns 64 tokens x 64 outputs of one head; its four warps take 16 tokens each and walk
// K in blocks of 32 through shared memory (rows padded to 40 entries: the fragment loads of a warp fall
// into 32 different banks).  Every output is one accumulator that walks k upwards, so a row's values do
// not depend on what else is in the batch.
#include "common.cuh"

using namespace fwb;

namespace {

constexpr int BM = 64, BN = 64, BK = 32, PAD = 8, LDS = BK + PAD;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// VEC: entries per global load (8: 16-byte loads, every row block starts on 16 bytes; 2: 4-byte loads).
template <int VEC>
__global__ void __launch_bounds__(128)
head_linear_mma_kernel(const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ W,
                       __nv_bfloat16* __restrict__ Y, int M, int N, int K, long long ldx, long long x_head,
                       long long ldy, long long y_head) {
    fwb::pdl_entry();
    __shared__ __align__(16) __nv_bfloat16 xs[BM][LDS];
    __shared__ __align__(16) __nv_bfloat16 ws[BN][LDS];
    const int h = blockIdx.z;
    X += (size_t)h * x_head;
    Y += (size_t)h * y_head;
    W += (size_t)h * N * K;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    float acc[BN / 8][4];
#pragma unroll
    for (int n = 0; n < BN / 8; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[n][j] = 0.0f;

    constexpr int PER_ROW = BK / VEC;                       // loads per tile row
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int i = threadIdx.x; i < BM * PER_ROW; i += 128) {
            const int r = i / PER_ROW, c = (i - r * PER_ROW) * VEC;
            const int k = k0 + c;
            if (VEC == 8) {
                uint4 xv = make_uint4(0u, 0u, 0u, 0u), wv = make_uint4(0u, 0u, 0u, 0u);
                if (m0 + r < M && k < K) xv = *reinterpret_cast<const uint4*>(X + (size_t)(m0 + r) * ldx + k);
                if (n0 + r < N && k < K) wv = *reinterpret_cast<const uint4*>(W + (size_t)(n0 + r) * K + k);
                *reinterpret_cast<uint4*>(&xs[r][c]) = xv;
                *reinterpret_cast<uint4*>(&ws[r][c]) = wv;
            } else {
                uint32_t xv = 0u, wv = 0u;
                if (m0 + r < M && k < K) xv = *reinterpret_cast<const uint32_t*>(X + (size_t)(m0 + r) * ldx + k);
                if (n0 + r < N && k < K) wv = *reinterpret_cast<const uint32_t*>(W + (size_t)(n0 + r) * K + k);
                *reinterpret_cast<uint32_t*>(&xs[r][c]) = xv;
                *reinterpret_cast<uint32_t*>(&ws[r][c]) = wv;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk += 16) {
            uint32_t a[4];
            const __nv_bfloat16* row_lo = &xs[warp * 16 + g][kk + 2 * t];
            const __nv_bfloat16* row_hi = &xs[warp * 16 + g + 8][kk + 2 * t];
            a[0] = *reinterpret_cast<const uint32_t*>(row_lo);
            a[1] = *reinterpret_cast<const uint32_t*>(row_hi);
            a[2] = *reinterpret_cast<const uint32_t*>(row_lo + 8);
            a[3] = *reinterpret_cast<const uint32_t*>(row_hi + 8);
#pragma unroll
            for (int n = 0; n < BN / 8; ++n) {
                const __nv_bfloat16* col = &ws[n * 8 + g][kk + 2 * t];
                mma_bf16_16816(acc[n], a, *reinterpret_cast<const uint32_t*>(col),
                               *reinterpret_cast<const uint32_t*>(col + 8));
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int m = m0 + warp * 16 + g + 8 * half;
        if (m >= M) continue;
#pragma unroll
        for (int n = 0; n < BN / 8; ++n) {
            const int col = n0 + n * 8 + 2 * t;
            if (col < N) {
                __nv_bfloat162 v = __floats2bfloat162_rn(acc[n][2 * half], acc[n][2 * half + 1]);
                *reinterpret_cast<__nv_bfloat162*>(Y + (size_t)m * ldy + col) = v;
            }
        }
    }
}

}  // namespace

// X: rows `ldx` entries apart, head h at entry h * x_head; W: [heads][N][K]; Y likewise with ldy, y_head.
// All bfloat16.  Needs even N, K, row lengths and head offsets, and 4-byte aligned X, W, Y (pairs of
// entries are moved together); anything else is refused and runs the fp32-FMA kernel.
FWB_API int fwb_head_linear_mma(const void* X, const void* W, void* Y, int M, int N, int K, int heads,
                                long long ldx, long long x_head, long long ldy, long long y_head,
                                cudaStream_t stream) {
    if (M <= 0 || N <= 0 || heads <= 0) return FWB_OK;
    if (!X || !W || !Y || K <= 0) return FWB_BAD_ARGUMENT;
    if ((N | K | ldx | x_head | ldy | y_head) & 1) return FWB_UNSUPPORTED;
    if ((((uintptr_t)X | (uintptr_t)W | (uintptr_t)Y) & 3) != 0) return FWB_UNSUPPORTED;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, heads);
    if (grid.y > 65535 || grid.z > 65535) return FWB_TOO_LARGE;
    using bf = __nv_bfloat16;
    const bool wide = ((K | ldx | x_head) & 7) == 0 && (((uintptr_t)X | (uintptr_t)W) & 15) == 0;
    if (wide)
        fwb::pdl(head_linear_mma_kernel<8>, grid, 128, 0, stream)((const bf*)X, (const bf*)W, (bf*)Y, M, N, K, ldx,
                                                                  x_head, ldy, y_head);
    else
        fwb::pdl(head_linear_mma_kernel<2>, grid, 128, 0, stream)((const bf*)X, (const bf*)W, (bf*)Y, M, N, K, ldx,
                                                                  x_head, ldy, y_head);
    return fwb_launch_status();
}
