// Log-mel frontend: PCM -> normalised log-mel features [utterance, frame, 128] fp32, the input
// of the subsampling stage.  Replaces run_frontend (src/cuda/frontend.rs:230-316) and its kernels
// pk_sm89_frame_window / cuFFT R2C / pk_sm89_mel_log_sparse / pk_sm89_normalize_mel
// (kernels/sm89/frontend.cu:11-115); CPU definition: CpuMelFrontend::compute
// (src/frontend.rs:114-215).
//
// One CTA per frame does framing (pre-emphasis, centred 512-sample window), a 512-point
// radix-2 FFT in shared memory, the power spectrum and the sparse mel filters, so the framed
// signal and the spectrum never travel through HBM (the reference stores both).  A second
// kernel normalises every mel row over the valid frames in double precision.
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "pk100_internal.h"

namespace pk100 {

constexpr int kFft = 512;
constexpr int kFftBins = kFft / 2 + 1;
constexpr int kHop = 160;
constexpr int kMels = 128;
constexpr int kLogFft = 9;

__global__ void __launch_bounds__(256)
mel_frames_kernel(const float* __restrict__ samples, long long sample_stride, const int* __restrict__ sample_counts,
                  const float* __restrict__ window, const int* __restrict__ filter_offsets,
                  const int* __restrict__ filter_bins, const float* __restrict__ filter_values,
                  float* __restrict__ mel, int frame_cap, float preemphasis, float log_zero_guard) {
    __shared__ float re[kFft], im[kFft];
    __shared__ float tw_re[kFft / 2], tw_im[kFft / 2];
    __shared__ float power[kFftBins];
    const int tid = threadIdx.x;
    const int frame = blockIdx.x, utt = blockIdx.y;
    const int count = sample_counts[utt];
    const int frames = count > 0 ? count / kHop + 1 : 0;
    float* out = mel + (static_cast<size_t>(utt) * frame_cap + frame) * kMels;
    if (frame >= frames) {                         // beyond this utterance: zero rows
        if (tid < kMels) out[tid] = 0.0f;
        return;
    }
    const float* pcm = samples + static_cast<size_t>(utt) * sample_stride;
    // twiddles e^{-2 pi i k / 512}
    {
        float s, c;
        sincospif(-2.0f * static_cast<float>(tid) / static_cast<float>(kFft), &s, &c);
        tw_re[tid] = c;
        tw_im[tid] = s;
    }
    // framing in bit-reversed order (decimation in time)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int i = tid + half * 256;
        const int sample = frame * kHop + i - kFft / 2;
        float v = 0.0f;
        if (sample >= 0 && sample < count) {
            v = pcm[sample];
            if (sample > 0) v -= preemphasis * pcm[sample - 1];
        }
        const int rev = static_cast<int>(__brev(static_cast<unsigned>(i)) >> (32 - kLogFft));
        re[rev] = v * window[i];
        im[rev] = 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int stage = 0; stage < kLogFft; ++stage) {
        const int half_len = 1 << stage;
        const int pos = tid & (half_len - 1);
        const int left = ((tid >> stage) << (stage + 1)) + pos;
        const int right = left + half_len;
        const int tw = pos << (kLogFft - 1 - stage);
        const float wr = tw_re[tw], wi = tw_im[tw];
        const float xr = re[right], xi = im[right];
        const float pr = wr * xr - wi * xi, pi = wr * xi + wi * xr;
        const float lr = re[left], li = im[left];
        re[right] = lr - pr;
        im[right] = li - pi;
        re[left] = lr + pr;
        im[left] = li + pi;
        __syncthreads();
    }
    for (int b = tid; b < kFftBins; b += 256) power[b] = re[b] * re[b] + im[b] * im[b];
    __syncthreads();
    if (tid < kMels) {
        float sum = 0.0f;
        for (int i = filter_offsets[tid]; i < filter_offsets[tid + 1]; ++i)
            sum = fmaf(filter_values[i], power[filter_bins[i]], sum);
        out[tid] = logf(sum + log_zero_guard);
    }
}

// One CTA per (mel bin, utterance): mean and unbiased variance over the valid frames in
// double precision, rows at or beyond the valid count become zero (frontend.cu:64-115).
__global__ void __launch_bounds__(256)
mel_normalize_kernel(float* __restrict__ mel, const int* __restrict__ sample_counts, int frame_cap, float epsilon,
                     int* __restrict__ valid_out) {
    __shared__ double red[256];
    const int bin = blockIdx.x, utt = blockIdx.y, tid = threadIdx.x;
    const int count = sample_counts[utt];
    const int valid = count > 0 ? count / kHop : 0;
    const int frames = count > 0 ? valid + 1 : 0;
    if (bin == 0 && tid == 0 && valid_out != nullptr) valid_out[utt] = valid;
    float* col = mel + static_cast<size_t>(utt) * frame_cap * kMels + bin;
    auto block_sum = [&](double v) {
        red[tid] = v;
        __syncthreads();
        for (int w = 128; w > 0; w /= 2) {
            if (tid < w) red[tid] += red[tid + w];
            __syncthreads();
        }
        const double total = red[0];
        __syncthreads();
        return total;
    };
    double s = 0.0;
    for (int f = tid; f < valid; f += 256) s += static_cast<double>(col[static_cast<size_t>(f) * kMels]);
    const double mean = valid > 0 ? block_sum(s) / valid : (block_sum(0.0), 0.0);
    double q = 0.0;
    for (int f = tid; f < valid; f += 256) {
        const double d = static_cast<double>(col[static_cast<size_t>(f) * kMels]) - mean;
        q += d * d;
    }
    const double sq = block_sum(q);
    const double variance = valid > 1 ? sq / static_cast<double>(valid - 1) : 0.0;
    const double denominator = sqrt(variance) + static_cast<double>(epsilon);
    for (int f = tid; f < frames; f += 256) {
        float* p = col + static_cast<size_t>(f) * kMels;
        *p = f < valid ? static_cast<float>((static_cast<double>(*p) - mean) / denominator) : 0.0f;
    }
}

}  // namespace pk100

using namespace pk100;

extern "C" int pk100_mel_frames_for(int samples) { return samples > 0 ? samples / kHop + 1 : 0; }

extern "C" int pk100_mel_frontend(void* stream_v, const pk100_frontend_weights* w, const float* samples,
                                  int utterances, long long sample_stride, const int* sample_counts, float* mel,
                                  int frame_cap, int* valid_frames) {
    if (!w || !w->window || !w->filter_offsets || !w->filter_bins || !w->filter_values || !samples ||
        !sample_counts || !mel)
        return PK100_ERR_NULL;
    if (utterances == 0) return PK100_OK;
    if (utterances < 0 || frame_cap <= 0 || sample_stride <= 0) return PK100_ERR_SHAPE;
    // every frame a utterance of sample_stride samples can have must fit the output block
    if (sample_stride / kHop + 1 > frame_cap) return PK100_ERR_SHAPE;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    mel_frames_kernel<<<dim3(frame_cap, utterances), 256, 0, stream>>>(
        samples, sample_stride, sample_counts, w->window, w->filter_offsets, w->filter_bins, w->filter_values, mel,
        frame_cap, w->preemphasis, w->log_zero_guard);
    int rc = pk100_launch_status();
    if (rc != PK100_OK) return rc;
    mel_normalize_kernel<<<dim3(kMels, utterances), 256, 0, stream>>>(mel, sample_counts, frame_cap,
                                                                      w->normalize_epsilon, valid_frames);
    return pk100_launch_status();
}
