// Token selection on the device from float32 logits [rows, vocab].
//
// One block per row. A row with temperature 0 takes the first maximum
// (crates/stride-backend/src/sampler.rs:157-165). Otherwise the logits are
// divided by the temperature, a max-subtracted softmax is formed in float32
// (sampler.rs:169-183) and the token is drawn by inverse CDF with the uniform
// number that the host's generator supplies: the first index, in vocabulary
// order, at which the running sum of probabilities reaches u * total. A
// suppressed token (EOS below min_tokens, sampler.rs:81-86) counts as -inf.
// Top-k and nucleus cuts need a ranking and are done by the host sampler.
#include "common.cuh"

namespace stride {

constexpr int kSampleThreads = 256;

__device__ __forceinline__ float masked_logit(const float* row, int i, int banned, float inv_t) {
    return i == banned ? -INFINITY : row[i] * inv_t;
}

__global__ void __launch_bounds__(kSampleThreads)
sample_rows_kernel(const float* __restrict__ logits, int vocab, long long row_stride, const float* __restrict__ temperature,
                   const float* __restrict__ uniform, const int32_t* __restrict__ suppress, int32_t* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ float s_val[kSampleThreads];
    __shared__ int s_idx[kSampleThreads];
    __shared__ float scratch[32];
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* row = logits + static_cast<size_t>(r) * row_stride;
    const int banned = suppress ? suppress[r] : -1;
    const float t = temperature ? temperature[r] : 0.f;
    const float inv_t = t > 0.f ? 1.f / t : 1.f;

    // Each thread owns one contiguous segment, so that the prefix sums below
    // run in vocabulary order.
    const int per = (vocab + kSampleThreads - 1) / kSampleThreads;
    const int lo = min(tid * per, vocab), hi = min(lo + per, vocab);

    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = lo; i < hi; ++i) {
        const float v = masked_logit(row, i, banned, inv_t);
        if (best_i == 0x7fffffff || v > best) {
            best = v;
            best_i = i;
        }
    }
    s_val[tid] = best;
    s_idx[tid] = best_i;
    __syncthreads();
    for (int step = kSampleThreads / 2; step > 0; step >>= 1) {
        if (tid < step) {
            const float ov = s_val[tid + step];
            const int oi = s_idx[tid + step];
            // the larger value wins; on a tie the lower index (segments are ordered by thread)
            if (oi != 0x7fffffff && (s_idx[tid] == 0x7fffffff || ov > s_val[tid])) {
                s_val[tid] = ov;
                s_idx[tid] = oi;
            }
        }
        __syncthreads();
    }
    const float mx = s_val[0];
    const int arg = s_idx[0];
    if (!(t > 0.f)) {
        if (tid == 0) out[r] = arg;
        return;
    }
    if (!isfinite(mx)) {  // every logit is -inf: uniform over the vocabulary
        if (tid == 0) out[r] = min(static_cast<int>(uniform[r] * vocab), vocab - 1);
        return;
    }
    float seg = 0.f;
    for (int i = lo; i < hi; ++i) seg += expf(masked_logit(row, i, banned, inv_t) - mx);
    __syncthreads();
    s_val[tid] = seg;
    __syncthreads();
    // serial scan over 256 segment sums by one thread: in order, deterministic
    if (tid == 0) {
        float total = 0.f;
        for (int i = 0; i < kSampleThreads; ++i) total += s_val[i];
        const float target = uniform[r] * total;
        float run = 0.f;
        int owner = kSampleThreads - 1;
        for (int i = 0; i < kSampleThreads; ++i) {
            if (run + s_val[i] >= target && s_val[i] > 0.f) { owner = i; break; }
            run += s_val[i];
        }
        scratch[0] = target - run;
        s_idx[0] = owner;
    }
    __syncthreads();
    const int owner = s_idx[0];
    if (tid == owner) {
        float remaining = scratch[0];
        int pick = -1, last_positive = -1;
        for (int i = lo; i < hi; ++i) {
            const float p = expf(masked_logit(row, i, banned, inv_t) - mx);
            if (p > 0.f) last_positive = i;
            remaining -= p;
            if (remaining <= 0.f && p > 0.f) { pick = i; break; }
        }
        if (pick < 0) pick = last_positive >= 0 ? last_positive : arg;
        out[r] = pick;
    }
}

}  // namespace stride

extern "C" int stride_sample_rows(const float* logits, int rows, int vocab, long long row_stride, const float* temperature,
                                  const float* uniform, const int32_t* suppress, int32_t* out, cudaStream_t stream) {
    if (rows < 0 || vocab <= 0 || row_stride < vocab) return STRIDE_BAD_ARGUMENT;
    if (temperature != nullptr && uniform == nullptr) return STRIDE_BAD_ARGUMENT;
    if (rows == 0) return 0;
    stride::launch(stride::sample_rows_kernel, dim3(rows), dim3(stride::kSampleThreads), 0, stream, logits, vocab, row_stride, temperature, uniform, suppress, out);
    return STRIDE_LAUNCH_STATUS();
}
