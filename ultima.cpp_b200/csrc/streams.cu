// Several copies of the residual stream (hyper-connections): xs [S, T, width] in float32, S <= 8.
//
// A sublayer reads u = sum_s a[s] xs[s] through a norm and writes its result y back into every copy,
//     xs'[t] = sum_s mix[s, t] xs[s] + b[t] * y        (all copies at once from the old ones),
// with small learned tables a [S], b [S], mix [S, S] (indexed [from, to]).  Three kernels:
//   streams_fill        every copy starts as the embedding's output
//   streams_pass        one block a row: optionally the write of the sublayer that has just run (y is cleared
//                       behind the read), then optionally the read of the next one with its RMS norm:
//                       h = norm(sum_s a[s] xs[s]) * w; a null: the plain sum of the copies (the model's end).
//                       ``rows`` (optional) picks the rows that are read (no write then).
// All sums are float32 and taken in the order of s, so a row's result does not depend on the batch.
#include "common.cuh"

constexpr int MAX_STREAMS = 8;

struct StreamTables {
    float a[MAX_STREAMS];                 // read weights
    float b[MAX_STREAMS];                 // write weights of y
    float mix[MAX_STREAMS][MAX_STREAMS];  // [from][to]
};

__global__ void streams_fill_kernel(const float* __restrict__ x, float* __restrict__ xs, long long n, int S) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = x[i];
    for (int s = 0; s < S; ++s) xs[s * n + i] = v;
}

UB_API int ub_streams_fill(const float* x, float* xs, int n_rows, int width, int S, cudaStream_t st) {
    const long long n = (long long)n_rows * width;
    if (n <= 0) return 0;
    if (S < 1 || S > MAX_STREAMS) return UB_ERR_ARG;
    return (int)ub_launch_dependent(streams_fill_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, x, xs, n, S);
}

template <typename TO>
__global__ void streams_pass_kernel(float* __restrict__ xs, long long stream_stride, int S, const float* __restrict__ mix,
                                    const float* __restrict__ b, float* __restrict__ y, const float* __restrict__ a,
                                    int do_read, const float* __restrict__ w, const int* __restrict__ rows,
                                    TO* __restrict__ out, int width, float eps) {
    extern __shared__ float u_row[];                  // [width]: what the next sublayer reads, before the norm
    __shared__ float red[33];
    __shared__ StreamTables tb;
    pdl_trigger();
    if (threadIdx.x < S) {
        tb.a[threadIdx.x] = a ? a[threadIdx.x] : 1.0f;
        tb.b[threadIdx.x] = b ? b[threadIdx.x] : 0.f;
    }
    if (mix && threadIdx.x < S * S) tb.mix[threadIdx.x / S][threadIdx.x % S] = mix[threadIdx.x];
    pdl_wait();
    __syncthreads();
    const long long r = blockIdx.x;
    const long long src = rows ? rows[r] : r;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v[MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < MAX_STREAMS; ++s) v[s] = s < S ? xs[s * stream_stride + src * width + i] : 0.f;
        if (mix) {
            const float yv = y[src * width + i];
            float nv[MAX_STREAMS];
#pragma unroll
            for (int t = 0; t < MAX_STREAMS; ++t) {
                float acc = 0.f;
#pragma unroll
                for (int s = 0; s < MAX_STREAMS; ++s) if (s < S) acc = fmaf(tb.mix[s][t], v[s], acc);
                nv[t] = fmaf(tb.b[t], yv, acc);
            }
#pragma unroll
            for (int t = 0; t < MAX_STREAMS; ++t) if (t < S) { v[t] = nv[t]; xs[t * stream_stride + src * width + i] = nv[t]; }
            y[src * width + i] = 0.f;
        }
        if (do_read) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s) if (s < S) u = fmaf(tb.a[s], v[s], u);
            u_row[i] = u;
            ss += u * u;
        }
    }
    if (!do_read) return;
    ss = block_sum(ss, red);
    const float inv = w ? inv_rms(ss, (float)width, eps) : 1.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        out[r * width + i] = from_f32<TO>(w ? u_row[i] * w[i] * inv : u_row[i]);
}

// mix, b, y: the write (all three or none); do_read: the read into ``out`` (a null: plain sum; w null: no norm).
UB_API int ub_streams_pass(float* xs, long long stream_stride, int S, const float* mix, const float* b, float* y,
                           const float* a, int do_read, const float* w, const int* rows, void* out, int out_dtype,
                           int n_rows, int width, float eps, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    if (S < 1 || S > MAX_STREAMS || width <= 0) return UB_ERR_ARG;
    if ((mix != nullptr) != (y != nullptr) || (mix != nullptr) != (b != nullptr)) return UB_ERR_ARG;
    if (mix && rows) return UB_ERR_ARG;
    if (!mix && !do_read) return 0;
    const size_t smem = do_read ? (size_t)width * sizeof(float) : 0;
    if (smem > 160 * 1024) return UB_ERR_ARG;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    cudaError_t e;
#define GO(TO) do { \
        if (smem > 48 * 1024) cudaFuncSetAttribute(streams_pass_kernel<TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        e = ub_launch_dependent(streams_pass_kernel<TO>, dim3(n_rows), dim3(threads), smem, st, xs, stream_stride, S, mix, b, y, a, \
                                do_read, w, rows, (TO*)out, width, eps); } while (0)
    if (out_dtype == UB_F32) GO(float);
    else if (out_dtype == UB_BF16) GO(__nv_bfloat16);
    else return UB_ERR_UNSUPPORTED;
#undef GO
    return (int)e;
}
