// Attention over a cached low-rank latent (one latent row per token, shared by every head).
//
// What the cache holds per token is one row  [ c (rank) | r (rot) | 0-padding ]  of `row` entries:
// c, the RMS-normed latent, and r, the rotated key part that all heads share.  Per head h the key is
// (U_h c | r) and the value V_h c.  The kernels here work on the latent directly:
//
//   score_h(i, j) = scale * ( (U_h^T q_h,plain) . c_j  +  q_h,rot . r_j )
//   out_h(i)      = V_h * sum_j p_h(i, j) c_j
//
// so a query head becomes one row  [ U_h^T q_plain | q_rot | 0 ]  of the same layout as a cache row,
// attention is "many query heads, one key head" whose values are the first `rank` columns of the key,
// and the two per-head products (U_h^T in front, V_h behind) are batched small matrix products
// (fwb_head_linear).  The softmax denominator also holds exp(sink_h): a key of score sink_h (not
// scaled) with a zero value, which is how the running maximum and sum are started.
//
// Kernels of this file:
//   fwb_latent_prepare    rotation of the queries' rotated part, RMS norm of the latent, rotation of
//                         the shared key part, write of the cache row (one pass over the projection)
//   fwb_head_linear       Y[t][h] = W[h] X[t][h] for every head, fp32 FMA (any sizes, any strides)
//   fwb_latent_attention_simt   the attention in fp32 arithmetic, any sizes: the 32-bit path
// In bfloat16 the per-head products run on tensor cores (head_linear_mma.cu) and the attention on the
// paged attention kernels (attention_tcgen05.cu, attention_mma.cu: one pool head that every query head
// reads, its rows keys and values at once, a sink per head).
#include "common.cuh"

using namespace fwb;

namespace {

// ------------------------------------------------------------------ prepare
// One block per token.  proj: [T][ld] rows that hold the queries at column 0 (per head: `dim` plain
// channels, then `rot` rotated ones) and, with a cache row to write, the latent projection
// (rank + rot entries) at column kv_col.  qa: [T][heads][row]; this kernel fills [rank, row) of every
// head (rotated part, zero padding), the per-head product fills [0, rank) afterwards.
// table: [positions][rot_dims/2][2] (cos, sin); the first rot_dims channels of a rotated part turn,
// pair i = channels (i, i + rot_dims/2) or (2i, 2i+1).
template <typename TP, typename TC>
__global__ void latent_prepare_kernel(const TP* __restrict__ proj, int ld, int kv_col,
                                      const float* __restrict__ norm_w, const float* __restrict__ table,
                                      const int* __restrict__ positions, const int* __restrict__ tok_seg,
                                      const int* __restrict__ block_table, int max_pages, int page_size,
                                      TP* __restrict__ qa, TC* __restrict__ pool, int heads, int dim, int rot,
                                      int rot_dims, int interleaved, int rank, int row, float eps) {
    fwb::pdl_entry();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = rot_dims >> 1;
    const float* cs = table + (size_t)pos * (half > 0 ? half : 1) * 2;
    const TP* src = proj + (size_t)t * ld;
    // where channel c of a rotated part comes from: (value, partner, sign of the sine term)
    auto turned = [&](const TP* part, int c) -> float {
        if (c >= rot_dims) return to_f32<TP>(part[c]);
        int pair, partner;
        float sign;
        if (interleaved) {
            pair = c >> 1;
            partner = c ^ 1;
            sign = (c & 1) ? 1.0f : -1.0f;
        } else {
            pair = c < half ? c : c - half;
            partner = c < half ? c + half : c - half;
            sign = c < half ? -1.0f : 1.0f;
        }
        const float co = cs[2 * pair], si = cs[2 * pair + 1];
        return to_f32<TP>(part[c]) * co + sign * to_f32<TP>(part[partner]) * si;
    };
    const int tail = row - rank;                     // rotated part + padding
    for (int i = threadIdx.x; i < heads * tail; i += blockDim.x) {
        const int h = i / tail, c = i - h * tail;
        const TP* part = src + (size_t)h * (dim + rot) + dim;
        qa[((size_t)t * heads + h) * row + rank + c] = from_f32<TP>(c < rot ? turned(part, c) : 0.0f);
    }
    if (!pool) return;
    const TP* lat = src + kv_col;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        const float v = to_f32<TP>(lat[c]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)rank + eps);
    const int page = block_table[(size_t)tok_seg[t] * max_pages + pos / page_size];
    TC* dst = pool + ((size_t)page * page_size + (pos % page_size)) * row;
    for (int c = threadIdx.x; c < row; c += blockDim.x) {
        float v = 0.0f;
        if (c < rank) v = (to_f32<TP>(lat[c]) * inv) * norm_w[c];
        else if (c < rank + rot) v = turned(lat + rank, c - rank);
        dst[c] = from_f32<TC>(v);
    }
}

// ------------------------------------------------------------------ per-head products
// Y[t*ldy + h*y_head + n] = sum_k W[h][n][k] * X[t*ldx + h*x_head + k]; W: [heads][N][K] contiguous.
// One accumulator per output walks k upwards, so a value does not depend on the batch.
constexpr int TM = 64, TN = 64, TK = 16;

template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(256)
head_linear_kernel(const TX* __restrict__ X, const TW* __restrict__ W, TY* __restrict__ Y, int M, int N,
                   int K, long long ldx, long long x_head, long long ldy, long long y_head) {
    fwb::pdl_entry();
    __shared__ float xs[TK][TM + 4];
    __shared__ float ws[TK][TN + 4];
    const int h = blockIdx.z;
    X += (size_t)h * x_head;
    Y += (size_t)h * y_head;
    W += (size_t)h * N * K;
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
    const int lrow = tid / 4, lk = (tid % 4) * 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            const int m = m0 + lrow, n = n0 + lrow;
            xs[lk + j][lrow] = (m < M && k < K) ? to_f32<TX>(X[(size_t)m * ldx + k]) : 0.0f;
            ws[lk + j][lrow] = (n < N && k < K) ? to_f32<TW>(W[(size_t)n * K + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[k][tm + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[k][tn + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + tm + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tn + j;
            if (n < N) Y[(size_t)m * ldy + n] = from_f32<TY>(acc[i][j]);
        }
    }
}

// ------------------------------------------------------------------ attention, fp32 arithmetic
// One block per (token, set of up to 16 heads).  The block walks the token's keys 0..pos in tiles
// of 32 rows that start at multiples of 32 (never across a page), stages a tile in shared memory
// once for all its heads, and lets every warp run an online softmax for its heads: lane = key for
// the scores, lane = latent channel for the weighted sum.  The walk depends on the token's own
// position only.
constexpr int WARPS = 4;
constexpr int TILE = 32;
constexpr int MAX_HPW = 4;    // heads per warp: 16 heads per block
constexpr int MAX_CPL = 16;   // latent channels per lane: rank <= 512

template <typename TQ, typename TC, typename TO>
__global__ void __launch_bounds__(WARPS * 32)
latent_attention_simt_kernel(const TQ* __restrict__ qa, const TC* __restrict__ pool,
                             const float* __restrict__ sink, const int* __restrict__ positions,
                             const int* __restrict__ tok_seg, const int* __restrict__ block_table,
                             int max_pages, int page_size, TO* __restrict__ out, int heads, int rank,
                             int used, int row, float scale) {
    fwb::pdl_entry();
    extern __shared__ float smem[];
    const int t = blockIdx.x, h0 = blockIdx.y * WARPS * MAX_HPW;
    const int mine = heads - h0 < WARPS * MAX_HPW ? heads - h0 : WARPS * MAX_HPW;
    float* qs = smem;                          // [mine][used]
    float* ks = qs + WARPS * MAX_HPW * used;   // [TILE][used + 1]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = positions[t];
    const int* table = block_table + (size_t)tok_seg[t] * max_pages;
    for (int i = threadIdx.x; i < mine * used; i += blockDim.x) {
        const int h = i / used, c = i - h * used;
        qs[i] = to_f32<TQ>(qa[((size_t)t * heads + h0 + h) * row + c]);
    }
    float m[MAX_HPW], l[MAX_HPW], acc[MAX_HPW][MAX_CPL];
#pragma unroll
    for (int a = 0; a < MAX_HPW; ++a) {
        const int h = warp + a * WARPS;
        // the sink: a key of score sink_h whose value is zero
        m[a] = (sink && h < mine) ? sink[h0 + h] : -INFINITY;
        l[a] = (sink && h < mine) ? 1.0f : 0.0f;
#pragma unroll
        for (int d = 0; d < MAX_CPL; ++d) acc[a][d] = 0.0f;
    }
    for (int base = 0; base <= pos; base += TILE) {
        __syncthreads();
        const int page = table[base / page_size];
        const TC* src = pool + ((size_t)page * page_size + (base % page_size)) * row;
        const int valid = pos - base + 1 < TILE ? pos - base + 1 : TILE;
        for (int i = threadIdx.x; i < TILE * used; i += blockDim.x) {
            const int r = i / used, c = i - r * used;
            ks[r * (used + 1) + c] = r < valid ? to_f32<TC>(src[(size_t)r * row + c]) : 0.0f;
        }
        __syncthreads();
        const bool seen = lane < valid;
#pragma unroll
        for (int a = 0; a < MAX_HPW; ++a) {
            const int h = warp + a * WARPS;
            if (h >= mine) break;
            const float* qh = qs + h * used;
            const float* kr = ks + lane * (used + 1);
            float s = 0.0f;
            for (int d = 0; d < used; ++d) s = fmaf(qh[d], kr[d], s);
            s = seen ? s * scale : -INFINITY;
            const float m_new = fmaxf(m[a], warp_max(s));
            const float p = seen ? expf(s - m_new) : 0.0f;
            const float corr = expf(m[a] - m_new);     // m == -inf (no sink, first tile) gives 0
            l[a] = l[a] * corr + warp_sum(p);
            m[a] = m_new;
#pragma unroll
            for (int d = 0; d < MAX_CPL; ++d) acc[a][d] *= corr;
            for (int j = 0; j < valid; ++j) {
                const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
                for (int d = 0; d < MAX_CPL; ++d) {
                    const int c = lane + 32 * d;
                    if (c < rank) acc[a][d] = fmaf(pj, ks[j * (used + 1) + c], acc[a][d]);
                }
            }
        }
    }
#pragma unroll
    for (int a = 0; a < MAX_HPW; ++a) {
        const int h = warp + a * WARPS;
        if (h >= mine) break;
        const float inv = 1.0f / l[a];
        TO* dst = out + ((size_t)t * heads + h0 + h) * rank;
#pragma unroll
        for (int d = 0; d < MAX_CPL; ++d) {
            const int c = lane + 32 * d;
            if (c < rank) dst[c] = from_f32<TO>(acc[a][d] * inv);
        }
    }
}

}  // namespace

// proj: [T][ld] (fp32 or bf16); qa: [T][heads][row] in proj's dtype; pool: [pages][page_size][row]
// (null: queries only; its dtype flag may differ from proj's), block_table: [S][max_pages].
FWB_API int fwb_latent_prepare(const void* proj, int proj_bf16, int ld, int kv_col, const float* norm_w,
                               const float* table, const int* positions, const int* tok_seg,
                               const int* block_table, int max_pages, int page_size, void* qa, void* pool,
                               int pool_bf16, int T, int heads, int dim, int rot, int rot_dims,
                               int interleaved, int rank, int row, float eps, cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!proj || !table || !positions || !qa) return FWB_BAD_ARGUMENT;
    if (heads <= 0 || dim < 0 || rot < 0 || rank <= 0 || row < rank + rot || rot_dims < 0 || rot_dims > rot
        || (rot_dims & 1) || ld < heads * (dim + rot))
        return FWB_BAD_ARGUMENT;
    if (pool && (!norm_w || !tok_seg || !block_table || max_pages <= 0 || page_size <= 0
                 || kv_col < heads * (dim + rot) || ld < kv_col + rank + rot))
        return FWB_BAD_ARGUMENT;
    using bf = __nv_bfloat16;
    const int threads = 128;
#define FWB_PREP(TP, TC)                                                                               \
    fwb::pdl(latent_prepare_kernel<TP, TC>, T, threads, 0, stream)(                                    \
        (const TP*)proj, ld, kv_col, norm_w, table, positions, tok_seg, block_table, max_pages,       \
        page_size, (TP*)qa, (TC*)pool, heads, dim, rot, rot_dims, interleaved, rank, row, eps)
    if (proj_bf16 && (pool_bf16 || !pool)) FWB_PREP(bf, bf);
    else if (!proj_bf16 && (!pool_bf16 || !pool)) FWB_PREP(float, float);
    else if (proj_bf16) FWB_PREP(bf, float);
    else FWB_PREP(float, bf);
#undef FWB_PREP
    return fwb_launch_status();
}

// X: rows `ldx` apart, head h at offset h * x_head; W: [heads][N][K]; Y likewise with ldy, y_head.
// Dtype flags: 0 fp32, 1 bf16 (all three equal).
FWB_API int fwb_head_linear(const void* X, const void* W, void* Y, int bf16, int M, int N, int K, int heads,
                            long long ldx, long long x_head, long long ldy, long long y_head,
                            cudaStream_t stream) {
    if (M <= 0 || N <= 0 || heads <= 0) return FWB_OK;
    if (!X || !W || !Y || K <= 0) return FWB_BAD_ARGUMENT;
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM, heads);
    if (grid.y > 65535 || grid.z > 65535) return FWB_TOO_LARGE;
    using bf = __nv_bfloat16;
    if (bf16)
        fwb::pdl(head_linear_kernel<bf, bf, bf>, grid, 256, 0, stream)((const bf*)X, (const bf*)W, (bf*)Y, M, N, K,
                                                                    ldx, x_head, ldy, y_head);
    else
        fwb::pdl(head_linear_kernel<float, float, float>, grid, 256, 0, stream)(
            (const float*)X, (const float*)W, (float*)Y, M, N, K, ldx, x_head, ldy, y_head);
    return fwb_launch_status();
}

// qa: [T][heads][row]; pool: [pages][page_size][row]; sink: fp32 [heads] or null; out: [T][heads][rank].
// `used` = rank + rot: the columns of a row that enter a score.
FWB_API int fwb_latent_attention_simt(const void* qa, const void* pool, int bf16, const float* sink,
                                      const int* positions, const int* tok_seg, const int* block_table,
                                      int max_pages, int page_size, void* out, int T, int heads, int rank,
                                      int used, int row, float scale, cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!qa || !pool || !positions || !tok_seg || !block_table || !out) return FWB_BAD_ARGUMENT;
    if (heads <= 0 || rank <= 0 || used < rank || row < used || max_pages <= 0) return FWB_BAD_ARGUMENT;
    if (page_size <= 0 || page_size % TILE != 0) return FWB_UNSUPPORTED;
    if (rank > 32 * MAX_CPL) return FWB_TOO_LARGE;
    const size_t smem = ((size_t)WARPS * MAX_HPW * used + (size_t)TILE * (used + 1)) * sizeof(float);
    if (smem > 200 * 1024) return FWB_TOO_LARGE;
    dim3 grid(T, (heads + WARPS * MAX_HPW - 1) / (WARPS * MAX_HPW));
    using bf = __nv_bfloat16;
#define FWB_LATENT(TT)                                                                                  \
    do {                                                                                                \
        auto kernel = latent_attention_simt_kernel<TT, TT, TT>;                                         \
        if (smem > 48 * 1024) {                                                                         \
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                                 (int)smem);                                            \
            if (e != cudaSuccess) return (int)e;                                                        \
        }                                                                                               \
        fwb::pdl(kernel, grid, WARPS * 32, smem, stream)((const TT*)qa, (const TT*)pool, sink, positions, \
                                                         tok_seg, block_table, max_pages, page_size,   \
                                                         (TT*)out, heads, rank, used, row, scale);      \
    } while (0)
    if (bf16) FWB_LATENT(bf);
    else FWB_LATENT(float);
#undef FWB_LATENT
    return fwb_launch_status();
}
