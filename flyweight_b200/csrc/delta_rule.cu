// The gated delta rule: a recurrent mixer whose per-request state is one [d][e] matrix per head.
//
// Per token and head, with unit vectors q (times d^-1/2) and k of size d, a value v of size e, a
// write strength beta in (0, 1) and a decay g in (0, 1):
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// so the read-out sees the token's own write.  q, k and v come from one fused projection
//     p[t] = [ q: G d | k: G d | v: H e | gate: H e | b: H | a: H ]        (fp32)
// through a short causal convolution over time per channel (taps [C][L], the last tap on the token
// itself) and silu; q and k are then made unit vectors per head (x / sqrt(sum x^2 + 1e-6)); query
// head h uses q/k head h / (H / G).  beta = sigmoid(b), g = exp(-exp(A_log) softplus(a + dt_bias)).
//
// Three kernels (everything fp32):
//   delta_prepare   one block per token: convolution + silu, unit vectors, beta and g
//                   -> r[t] = [ q^: G d | k^: G d | v: H e | beta: H | g: H | q^.k^: G ]
//   delta_scan      one block per (16 or 32 columns of S, head, segment): the recurrence over the
//                   segment's tokens in order.  A column of S evolves independently of the others;
//                   four or eight adjacent lanes hold one column in registers, so a token costs two
//                   reductions over those lanes.  State in and out of the request's slot.  The first
//                   block of a segment also moves the convolution's last L-1 inputs on, for the next
//                   step (behind delta_prepare, which reads the old ones).
//   gated_head_norm out[t][h] = weight * o / sqrt(mean(o^2) + eps) * silu(gate)
// A request's slot is [ S: H d e | conv inputs: C (L-1) ] fp32, zero when the request starts.  A
// token's result depends on its request's earlier tokens only through that slot, and every sum runs
// in an order fixed by the sizes, so it does not depend on how the sequence was cut into steps.
#include "common.cuh"

using namespace fwb;

namespace {

constexpr int MAX_TAPS = 16;

struct DeltaShape {
    int H, G, d, e, L;      // heads, q/k heads, q/k size, value size, taps
    __host__ __device__ int cq() const { return G * d; }
    __host__ __device__ int cv() const { return H * e; }
    __host__ __device__ int channels() const { return 2 * G * d + H * e; }      // through the convolution
    __host__ __device__ int p_width() const { return channels() + H * e + 2 * H; }
    // (rows of r are padded to 16 bytes, so that 16-byte copies may start at a head's first channel)
    __host__ __device__ int r_width() const { return (channels() + 2 * H + G + 3) & ~3; }
};

__global__ void __launch_bounds__(512)
delta_prepare_kernel(const float* __restrict__ p, const float* __restrict__ taps, const float* __restrict__ a_log,
                     const float* __restrict__ dt_bias, const float* __restrict__ state, long long slot_stride,
                     const int* __restrict__ seg_start, const int* __restrict__ seg_slot,
                     const int* __restrict__ tok_seg, float* __restrict__ r, DeltaShape sh) {
    fwb::pdl_entry();
    extern __shared__ float c[];                  // the token's channels behind convolution and silu
    const int t = blockIdx.x;
    const int seg = tok_seg[t];
    const int local = t - seg_start[seg];         // tokens of this request in front of t in this step
    const int C = sh.channels(), P = sh.p_width(), R = sh.r_width(), L = sh.L;
    const float* hist = state + (size_t)seg_slot[seg] * slot_stride + (size_t)sh.H * sh.d * sh.e;
    for (int ch = threadIdx.x; ch < C; ch += blockDim.x) {
        float acc = 0.0f;
        for (int j = 0; j < L; ++j) {
            const int back = L - 1 - j;           // tap j multiplies the input `back` tokens ago
            const float x = back <= local ? p[(size_t)(t - back) * P + ch]
                                          : hist[(size_t)ch * (L - 1) + (L - 1) - (back - local)];
            acc = fmaf(taps[(size_t)ch * L + j], x, acc);
        }
        c[ch] = silu_f32(acc);
    }
    __syncthreads();
    float* out = r + (size_t)t * R;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const float q_scale = rsqrtf((float)sh.d);
    for (int head = warp; head < sh.G; head += warps) {            // query head and key head `head` together
        const float* q = c + (size_t)head * sh.d;
        const float* k = c + (size_t)(sh.G + head) * sh.d;
        float qq = 0.0f, kk = 0.0f, qk = 0.0f;
        for (int i = lane; i < sh.d; i += 32) {
            qq = fmaf(q[i], q[i], qq);
            kk = fmaf(k[i], k[i], kk);
            qk = fmaf(q[i], k[i], qk);
        }
        qq = warp_sum(qq), kk = warp_sum(kk), qk = warp_sum(qk);
        const float inv_q = (1.0f / sqrtf(qq + 1e-6f)) * q_scale, inv_k = 1.0f / sqrtf(kk + 1e-6f);
        for (int i = lane; i < sh.d; i += 32) {
            out[(size_t)head * sh.d + i] = q[i] * inv_q;
            out[(size_t)(sh.G + head) * sh.d + i] = k[i] * inv_k;
        }
        if (lane == 0) out[C + 2 * sh.H + head] = (qk * inv_q) * inv_k;      // q^ . k^, for the read-out
    }
    for (int i = threadIdx.x; i < sh.cv(); i += blockDim.x) out[2 * sh.cq() + i] = c[2 * sh.cq() + i];
    for (int h = threadIdx.x; h < sh.H; h += blockDim.x) {
        const float b = p[(size_t)t * P + C + sh.cv() + h];
        const float a = p[(size_t)t * P + C + sh.cv() + sh.H + h] + dt_bias[h];
        const float softplus = a > 20.0f ? a : log1pf(expf(a));
        out[C + h] = 1.0f / (1.0f + expf(-b));
        out[C + sh.H + h] = expf(-expf(a_log[h]) * softplus);
    }
}

// The request's last L-1 inputs of every channel, for the next step.  Runs in the kernel behind
// delta_prepare (which reads the old ones): the first block of every segment's scan does it.
__device__ __forceinline__ void delta_conv_advance(const float* __restrict__ p, float* __restrict__ slot, int t0,
                                                   int n, const DeltaShape& sh) {
    const int keep = sh.L - 1, P = sh.p_width();
    for (int ch = threadIdx.x; ch < sh.channels(); ch += blockDim.x) {
        float* hist = slot + (size_t)sh.H * sh.d * sh.e + (size_t)ch * keep;
        float next[MAX_TAPS];
        for (int j = 0; j < keep; ++j) {
            const int local = n - keep + j;       // the input that becomes entry j (oldest first)
            next[j] = local >= 0 ? p[(size_t)(t0 + local) * P + ch] : hist[j + n];
        }
        for (int j = 0; j < keep; ++j) hist[j] = next[j];
    }
}

__device__ __forceinline__ void copy_async_f32(float* dst_shared, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_shared)), "l"(src)
                 : "memory");
}
__device__ __forceinline__ void copy_async_16(float* dst_shared, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_shared)), "l"(src)
                 : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// LPC adjacent lanes hold one column of S, DPL consecutive entries each (LPC * DPL >= d).  The tokens'
// q, k, v, beta, g and q.k arrive through a ring of asynchronous copies that runs three tokens ahead of the
// arithmetic.  Per token both sums over the *old* column, a = S.k and b = S.q, are taken in one pass and
// reduced over the LPC lanes together; then
//     u = beta (v - g a),   o = g b + u (q.k),   S <- g S + k u
// which is the recurrence in the order the header states (the read-out sees the token's write), with
// one reduction on the way to the next token instead of two.  In a slot, S lies column by column:
// S[h][column][d].  VEC: d and e are multiples of 4 and slots start on 16-byte borders: copies and
// state accesses of 16 bytes.
template <int DPL, int LPC, bool VEC>
__global__ void __launch_bounds__(128)
delta_scan_kernel(const float* __restrict__ r, const float* __restrict__ p, float* __restrict__ state,
                  long long slot_stride, const int* __restrict__ seg_start, const int* __restrict__ seg_slot,
                  float* __restrict__ o, DeltaShape sh) {
    // The next kernel is released only behind the token loop: its blocks would otherwise sit on the SMs for
    // the whole scan, whose one warp a scheduler is slowed by every other resident warp.
    fwb::pdl_wait();
    constexpr int COLS = 128 / LPC, STRIDE = DPL + 4, STAGES = 4;     // (+4: lanes' float4 reads hit apart banks)
    constexpr int KQ = 2 * LPC * STRIDE;                              // floats of one stage's k and q
    __shared__ __align__(16) float kq[STAGES][KQ];
    __shared__ __align__(16) float vs[STAGES][COLS];
    __shared__ float scalars[STAGES][4];                              // beta, g, q.k
    const int seg = blockIdx.z, h = blockIdx.y;
    const int t0 = seg_start[seg], t1 = seg_start[seg + 1];
    if (t1 <= t0) return;
    const int d = sh.d, e = sh.e, R = sh.r_width();
    const int kv_head = h / (sh.H / sh.G);
    const int col_local = threadIdx.x / LPC, sub = threadIdx.x % LPC;
    const int col = blockIdx.x * COLS + col_local;
    const bool valid = col < e;
    float* slot = state + (size_t)seg_slot[seg] * slot_stride;
    if (blockIdx.x == 0 && h == 0 && sh.L > 1) delta_conv_advance(p, slot, t0, t1 - t0, sh);
    float* S_col = slot + ((size_t)h * e + (valid ? col : 0)) * d;
    float S[DPL];
    if (VEC) {
#pragma unroll
        for (int i = 0; i < DPL; i += 4) {
            const int dd = sub * DPL + i;
            const float4 v = (valid && dd < d) ? *reinterpret_cast<const float4*>(S_col + dd) : make_float4(0.f, 0.f, 0.f, 0.f);
            S[i] = v.x, S[i + 1] = v.y, S[i + 2] = v.z, S[i + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int dd = sub * DPL + i;
            S[i] = (valid && dd < d) ? S_col[dd] : 0.0f;
        }
    }
    if (d < DPL * LPC || (int)(blockIdx.x + 1) * COLS > e) {
        // entries behind the head's last channel and columns behind the last are never copied: zeros
        for (int i = threadIdx.x; i < STAGES * KQ; i += blockDim.x) (&kq[0][0])[i] = 0.0f;
        for (int i = threadIdx.x; i < STAGES * COLS; i += blockDim.x) (&vs[0][0])[i] = 0.0f;
        __syncthreads();
    }
    const int q_at = kv_head * d, k_at = sh.cq() + kv_head * d, v_at = 2 * sh.cq() + h * e;
    // what this thread copies for every token (VEC): one 16-byte piece of k|q, the fourth warp's first
    // lanes the values, three lanes the token's scalars
    const int piece = threadIdx.x * 4;
    const bool has_piece = piece < 2 * d;
    const int piece_which = piece >= d ? 1 : 0, piece_dd = piece - piece_which * d;
    const int piece_src = (piece_which ? q_at : k_at) + piece_dd;
    const int piece_dst = piece_which * LPC * STRIDE + (piece_dd / DPL) * STRIDE + piece_dd % DPL;
    const int c4 = (threadIdx.x - 96) * 4;
    const bool has_v = threadIdx.x >= 96 && c4 < COLS && (int)blockIdx.x * COLS + c4 < e;
    const int v_src = v_at + blockIdx.x * COLS + c4;
    const int which_scalar = threadIdx.x - 120;                       // 0 beta, 1 g, 2 q.k
    const int scalar_src = which_scalar == 0 ? sh.channels() + h
                                             : (which_scalar == 1 ? sh.channels() + sh.H + h
                                                                  : sh.channels() + 2 * sh.H + kv_head);
    auto fetch = [&](int t, int stage) {
        if (t < t1) {
            const float* row = r + (size_t)t * R;
            if (VEC) {
                if (has_piece) copy_async_16(&kq[stage][piece_dst], row + piece_src);
                if (has_v) copy_async_16(&vs[stage][c4], row + v_src);
            } else {
                for (int i = threadIdx.x; i < 2 * d; i += blockDim.x) {
                    const int which = i >= d ? 1 : 0, dd = i - which * d;
                    copy_async_f32(&kq[stage][which * LPC * STRIDE + (dd / DPL) * STRIDE + dd % DPL],
                                   row + (which ? q_at : k_at) + dd);
                }
                if (threadIdx.x < COLS && blockIdx.x * COLS + threadIdx.x < e)
                    copy_async_f32(&vs[stage][threadIdx.x], row + v_at + blockIdx.x * COLS + threadIdx.x);
            }
            if (which_scalar >= 0 && which_scalar < 3) copy_async_f32(&scalars[stage][which_scalar], row + scalar_src);
        }
        copy_async_commit();
    };
    for (int j = 0; j < STAGES - 1; ++j) fetch(t0 + j, j);
    float* out_at = o + ((size_t)t0 * sh.H + h) * e + col;
    const size_t out_step = (size_t)sh.H * e;
    for (int t = t0; t < t1; ++t, out_at += out_step) {
        const int stage = (t - t0) % STAGES;
        copy_async_wait<STAGES - 2>();          // this token's copies have landed (mine; the barrier: everybody's)
        __syncthreads();                        // ... and everybody is done with the token before
        fetch(t + STAGES - 1, (t - t0 + STAGES - 1) % STAGES);
        const float beta = scalars[stage][0], g = scalars[stage][1], qk = scalars[stage][2];
        const float4* k4 = reinterpret_cast<const float4*>(&kq[stage][sub * STRIDE]);
        const float4* q4 = reinterpret_cast<const float4*>(&kq[stage][LPC * STRIDE + sub * STRIDE]);
        float a[4] = {0.0f, 0.0f, 0.0f, 0.0f}, b[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int i = 0; i < DPL / 4; ++i) {
            const float4 k = k4[i], q = q4[i];
            a[0] = fmaf(S[4 * i], k.x, a[0]), b[0] = fmaf(S[4 * i], q.x, b[0]);
            a[1] = fmaf(S[4 * i + 1], k.y, a[1]), b[1] = fmaf(S[4 * i + 1], q.y, b[1]);
            a[2] = fmaf(S[4 * i + 2], k.z, a[2]), b[2] = fmaf(S[4 * i + 2], q.z, b[2]);
            a[3] = fmaf(S[4 * i + 3], k.w, a[3]), b[3] = fmaf(S[4 * i + 3], q.w, b[3]);
        }
        float sk = (a[0] + a[1]) + (a[2] + a[3]), sq = (b[0] + b[1]) + (b[2] + b[3]);
#pragma unroll
        for (int offset = 1; offset < LPC; offset <<= 1) {
            sk += __shfl_xor_sync(0xffffffffu, sk, offset);
            sq += __shfl_xor_sync(0xffffffffu, sq, offset);
        }
        const float u = beta * (vs[stage][col_local] - g * sk);
        if (sub == 0 && valid) *out_at = fmaf(g, sq, u * qk);
#pragma unroll
        for (int i = 0; i < DPL / 4; ++i) {
            const float4 k = k4[i];
            S[4 * i] = fmaf(g, S[4 * i], k.x * u);
            S[4 * i + 1] = fmaf(g, S[4 * i + 1], k.y * u);
            S[4 * i + 2] = fmaf(g, S[4 * i + 2], k.z * u);
            S[4 * i + 3] = fmaf(g, S[4 * i + 3], k.w * u);
        }
    }
    copy_async_wait<0>();
    fwb::pdl_launch_dependents();
    if (VEC) {
#pragma unroll
        for (int i = 0; i < DPL; i += 4) {
            const int dd = sub * DPL + i;
            if (valid && dd < d) *reinterpret_cast<float4*>(S_col + dd) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
        }
    } else {
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int dd = sub * DPL + i;
            if (valid && dd < d) S_col[dd] = S[i];
        }
    }
}

template <typename TO>
__global__ void __launch_bounds__(128)
gated_head_norm_kernel(const float* __restrict__ o, const float* __restrict__ gate, long long gate_stride,
                       const float* __restrict__ weight, float eps, TO* __restrict__ out, int rows, int H, int e) {
    fwb::pdl_entry();
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const int t = row / H, h = row - t * H;
    const float* src = o + (size_t)row * e;
    const float* g = gate + (size_t)t * gate_stride + (size_t)h * e;
    float ss = 0.0f;
    for (int i = lane; i < e; i += 32) ss = fmaf(src[i], src[i], ss);
    const float inv = rsqrtf(warp_sum(ss) / (float)e + eps);
    for (int i = lane; i < e; i += 32)
        out[(size_t)row * e + i] = from_f32<TO>(((src[i] * inv) * weight[i]) * silu_f32(g[i]));
}

}  // namespace

// p: [T][2Gd + 2He + 2H] fp32 (q | k | v | gate | b | a).  taps: [2Gd + He][L] fp32.  a_log, dt_bias: [H].
// state: [slots][slot_stride] fp32 with S at 0 and the convolution's inputs behind it.
// r: [T][2Gd + He + 2H + G rounded up to a multiple of 4] fp32 scratch.  o: [T][H][e] fp32.
FWB_API int fwb_delta_rule(const float* p, const float* taps, const float* a_log, const float* dt_bias,
                           float* state, long long slot_stride, const int* seg_start, const int* seg_slot,
                           const int* tok_seg, float* r, float* o, int T, int n_segments, int H, int G, int d,
                           int e, int L, cudaStream_t stream) {
    if (T <= 0 || n_segments <= 0) return FWB_OK;
    if (!p || !taps || !a_log || !dt_bias || !state || !seg_start || !seg_slot || !tok_seg || !r || !o)
        return FWB_BAD_ARGUMENT;
    if (H <= 0 || G <= 0 || H % G || d <= 0 || e <= 0 || L < 1) return FWB_BAD_ARGUMENT;
    if (L > MAX_TAPS || d > 256) return FWB_TOO_LARGE;
    const DeltaShape sh{H, G, d, e, L};
    if (slot_stride < (long long)H * d * e + (long long)sh.channels() * (L - 1)) return FWB_BAD_ARGUMENT;
    const size_t smem = (size_t)sh.channels() * sizeof(float);
    if (smem > 160 * 1024 || n_segments > 65535 || H > 65535) return FWB_TOO_LARGE;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(delta_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int prepare_threads = sh.channels() >= 2048 ? 512 : (sh.channels() >= 512 ? 256 : 128);
    fwb::pdl(delta_prepare_kernel, T, prepare_threads, smem, stream)(p, taps, a_log, dt_bias, state, slot_stride,
                                                                     seg_start, seg_slot, tok_seg, r, sh);
    const bool vec = d % 4 == 0 && e % 4 == 0 && slot_stride % 4 == 0 && ((uintptr_t)state & 15) == 0 &&
                     ((uintptr_t)r & 15) == 0;
#define FWB_SCAN(DPL, LPC)                                                                                 \
    do {                                                                                                   \
        const dim3 grid((e + 128 / LPC - 1) / (128 / LPC), H, n_segments);                                 \
        if (vec)                                                                                           \
            fwb::pdl(delta_scan_kernel<DPL, LPC, true>, grid, 128, 0, stream)(r, p, state, slot_stride,    \
                                                                              seg_start, seg_slot, o, sh); \
        else                                                                                               \
            fwb::pdl(delta_scan_kernel<DPL, LPC, false>, grid, 128, 0, stream)(r, p, state, slot_stride,   \
                                                                               seg_start, seg_slot, o, sh); \
    } while (0)
    if (d <= 16) FWB_SCAN(4, 4);
    else if (d <= 32) FWB_SCAN(8, 4);
    else if (d <= 64) FWB_SCAN(16, 4);
    else if (d <= 128) FWB_SCAN(16, 8);
    else FWB_SCAN(32, 8);
#undef FWB_SCAN
    return fwb_launch_status();
}

// o: [T][H][e] fp32; gate: row t at gate + t * gate_stride, [H][e] fp32; weight: [e]; out: [T][H e].
FWB_API int fwb_gated_head_norm(const float* o, const float* gate, long long gate_stride, const float* weight,
                                float eps, void* out, int out_bf16, int T, int H, int e, cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!o || !gate || !weight || !out || H <= 0 || e <= 0) return FWB_BAD_ARGUMENT;
    const long long rows = (long long)T * H;
    if (rows > 2147483647LL / 4) return FWB_TOO_LARGE;
    const int blocks = (int)((rows + 3) / 4);
    if (out_bf16)
        fwb::pdl(gated_head_norm_kernel<__nv_bfloat16>, blocks, 128, 0, stream)(o, gate, gate_stride, weight, eps,
                                                                                 (__nv_bfloat16*)out, (int)rows, H, e);
    else
        fwb::pdl(gated_head_norm_kernel<float>, blocks, 128, 0, stream)(o, gate, gate_stride, weight, eps,
                                                                        (float*)out, (int)rows, H, e);
    return fwb_launch_status();
}
