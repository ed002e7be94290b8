// Operations on the fp32 residual stream that carry one token's worth of state from a step to
// the next: an embedding with a hashed table of token pairs (state: the request's last token), the
// token shift (state: the request's last row of the stream), and the residual sum behind a norm
// that has one gain for all channels.  All arithmetic is fp32; T only names a storage type.
//
// State and the cut of a batch: a request's tokens of a step are one segment.  The first token of
// a segment reads the state, every other token reads its left neighbour in the batch, and the
// thread that read the state is the one that stores the segment's last token (or row) into it
// afterwards, so nobody else touches that slot during the launch and the result does not depend
// on where a prompt was cut.
#include "common.cuh"

using namespace fwb;

namespace {

// ------------------------------------------------------------------ embedding + hashed pairs
// out[t] = scale * table[id_t] + pairs[row_t],  row_t = (id_{t-1} * mul_prev + id_t * mul_cur) mod
// buckets, and row `buckets` (the table's last) at position 0.
template <typename TW>
__global__ void embed_pair_hash_kernel(const TW* __restrict__ table, const TW* __restrict__ pairs,
                                       const int* __restrict__ ids, const int* __restrict__ positions,
                                       const int* __restrict__ tok_seg, const int* __restrict__ seg_start,
                                       const int* __restrict__ seg_slot, int* __restrict__ last_token,
                                       long long slot_stride, float* __restrict__ out, int W, int V,
                                       int buckets, long long mul_prev, long long mul_cur, int* bad,
                                       float scale) {
    fwb::pdl_entry();
    __shared__ long long pair_row;
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < V;
    if (threadIdx.x == 0) {
        const int seg = tok_seg[t];
        const int pos = positions[t];
        int before;
        if (t == seg_start[seg]) {
            int* slot = last_token + (long long)seg_slot[seg] * slot_stride;
            before = pos == 0 ? -1 : *slot;
            *slot = ids[seg_start[seg + 1] - 1];
        } else {
            before = ids[t - 1];
        }
        long long row = buckets;
        if (pos != 0) {
            row = ((long long)before * mul_prev + (long long)id * mul_cur) % (long long)buckets;
            if (row < 0) row += buckets;
        }
        pair_row = row;
        if (!ok && bad) atomicExch(bad, 1);
    }
    __syncthreads();
    const TW* row = table + (size_t)(ok ? id : 0) * W;
    const TW* extra = pairs + (size_t)pair_row * W;
    float* dst = out + (size_t)t * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x)
        dst[c] = ok ? fmaf(scale, to_f32<TW>(row[c]), to_f32<TW>(extra[c])) : 0.0f;
}

// ------------------------------------------------------------------ token shift
// out[t] = x[t] + (x[t-1] - x[t]) * mu, with x[-1] = 0 at position 0 and the request's last row of
// an earlier step at the head of a later portion.
template <typename TO>
__global__ void token_shift_kernel(const float* __restrict__ x, const float* __restrict__ mu,
                                   float* __restrict__ last_row, long long slot_stride,
                                   const int* __restrict__ positions, const int* __restrict__ tok_seg,
                                   const int* __restrict__ seg_start, const int* __restrict__ seg_slot,
                                   TO* __restrict__ out, int W) {
    fwb::pdl_entry();
    const int t = blockIdx.x;
    const int seg = tok_seg[t];
    const bool head = t == seg_start[seg];
    const float* cur = x + (size_t)t * W;
    TO* dst = out + (size_t)t * W;
    if (!head) {
        const float* before = cur - W;
        for (int c = threadIdx.x; c < W; c += blockDim.x) {
            const float v = cur[c];
            dst[c] = from_f32<TO>(fmaf(before[c] - v, mu[c], v));
        }
        return;
    }
    const bool first = positions[t] == 0;
    float* slot = last_row + (long long)seg_slot[seg] * slot_stride;
    const float* last = x + (size_t)(seg_start[seg + 1] - 1) * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = cur[c];
        const float before = first ? 0.0f : slot[c];
        slot[c] = last[c];
        dst[c] = from_f32<TO>(fmaf(before - v, mu[c], v));
    }
}

// ------------------------------------------------------------------ x += gain * unit(y)
// unit(y) = y / sqrt(mean(y^2) + eps); `copy` (optional) receives the new x in another dtype, for
// the matrix product that reads the stream next.
template <typename TC>
__global__ void unit_rms_gain_add_kernel(float* __restrict__ x, const float* __restrict__ y,
                                         const float* __restrict__ gain, TC* __restrict__ copy, int W,
                                         float eps) {
    fwb::pdl_entry();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const float* yr = y + (size_t)t * W;
    float* xr = x + (size_t)t * W;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) ss = fmaf(yr[c], yr[c], ss);
    ss = block_sum(ss, scratch);
    const float f = rsqrtf(ss / (float)W + eps) * gain[0];
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = fmaf(yr[c], f, xr[c]);
        xr[c] = v;
        if (copy) copy[(size_t)t * W + c] = from_f32<TC>(v);
    }
}

int threads_for(int W) {
    int threads = ((W + 31) / 32) * 32;
    return threads > 256 ? 256 : threads;
}

}  // namespace

// table: [V][W], pairs: [buckets + 1][W] (both fp32 or both bf16).  last_token: one int32 per state
// slot, `slot_stride` words apart.  ids, positions, tok_seg: [T]; seg_start: [S+1]; seg_slot: [S].
FWB_API int fwb_embed_pair_hash(const void* table, const void* pairs, int tables_bf16, const int* ids,
                                const int* positions, const int* tok_seg, const int* seg_start,
                                const int* seg_slot, int* last_token, long long slot_stride, float* out,
                                int T, int W, int V, int buckets, long long mul_prev, long long mul_cur,
                                int* bad, float scale, cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!table || !pairs || !ids || !positions || !tok_seg || !seg_start || !seg_slot || !last_token || !out)
        return FWB_BAD_ARGUMENT;
    if (W <= 0 || V <= 0 || buckets <= 0 || slot_stride <= 0) return FWB_BAD_ARGUMENT;
    if (tables_bf16)
        fwb::pdl(embed_pair_hash_kernel<__nv_bfloat16>, T, threads_for(W), 0, stream)(
            (const __nv_bfloat16*)table, (const __nv_bfloat16*)pairs, ids, positions, tok_seg, seg_start,
            seg_slot, last_token, slot_stride, out, W, V, buckets, mul_prev, mul_cur, bad, scale);
    else
        fwb::pdl(embed_pair_hash_kernel<float>, T, threads_for(W), 0, stream)(
            (const float*)table, (const float*)pairs, ids, positions, tok_seg, seg_start, seg_slot,
            last_token, slot_stride, out, W, V, buckets, mul_prev, mul_cur, bad, scale);
    return fwb_launch_status();
}

// x: fp32 [T][W]; mu: fp32 [W]; last_row: fp32 [slots][W], `slot_stride` floats apart; out: [T][W].
FWB_API int fwb_token_shift(const float* x, const float* mu, float* last_row, long long slot_stride,
                            const int* positions, const int* tok_seg, const int* seg_start,
                            const int* seg_slot, void* out, int out_bf16, int T, int W,
                            cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!x || !mu || !last_row || !positions || !tok_seg || !seg_start || !seg_slot || !out)
        return FWB_BAD_ARGUMENT;
    if (W <= 0 || slot_stride < W) return FWB_BAD_ARGUMENT;
    if (out_bf16)
        fwb::pdl(token_shift_kernel<__nv_bfloat16>, T, threads_for(W), 0, stream)(
            x, mu, last_row, slot_stride, positions, tok_seg, seg_start, seg_slot, (__nv_bfloat16*)out, W);
    else
        fwb::pdl(token_shift_kernel<float>, T, threads_for(W), 0, stream)(
            x, mu, last_row, slot_stride, positions, tok_seg, seg_start, seg_slot, (float*)out, W);
    return fwb_launch_status();
}

// x (in place), y: fp32 [T][W]; gain: one fp32 on the device; copy: null, or [T][W] bf16 / fp32.
FWB_API int fwb_unit_rms_gain_add(float* x, const float* y, const float* gain, void* copy, int copy_bf16,
                                  int T, int W, float eps, cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!x || !y || !gain || W <= 0) return FWB_BAD_ARGUMENT;
    if (copy_bf16)
        fwb::pdl(unit_rms_gain_add_kernel<__nv_bfloat16>, T, threads_for(W), 0, stream)(
            x, y, gain, (__nv_bfloat16*)copy, W, eps);
    else
        fwb::pdl(unit_rms_gain_add_kernel<float>, T, threads_for(W), 0, stream)(x, y, gain, (float*)copy, W, eps);
    return fwb_launch_status();
}
