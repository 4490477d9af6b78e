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

// The same pass four columns a thread (width a multiple of 4, S known when compiled): 16-byte loads and stores.
// Every element's sums are taken in the same order as in the kernel above.
template <typename TO, int SN>
__global__ void streams_pass_vec_kernel(float* __restrict__ xs, long long stream_stride, const float* __restrict__ mix,
                                        const float* __restrict__ b, float* __restrict__ y, const float* __restrict__ a,
                                        int do_read, const float* __restrict__ w, const int* __restrict__ rows,
                                        TO* __restrict__ out, int width, float eps) {
    extern __shared__ float4 u_row4[];                // [width / 4]
    __shared__ float red[33];
    __shared__ StreamTables tb;
    pdl_trigger();
    if (threadIdx.x < SN) {
        tb.a[threadIdx.x] = a ? a[threadIdx.x] : 1.0f;
        tb.b[threadIdx.x] = b ? b[threadIdx.x] : 0.f;
    }
    if (mix && threadIdx.x < SN * SN) tb.mix[threadIdx.x / SN][threadIdx.x % SN] = mix[threadIdx.x];
    pdl_wait();
    __syncthreads();
    const long long r = blockIdx.x;
    const long long src = rows ? rows[r] : r;
    const int w4 = width >> 2;
    float ss = 0.f;
    for (int i = threadIdx.x; i < w4; i += blockDim.x) {
        float4 v[SN];
#pragma unroll
        for (int s = 0; s < SN; ++s) v[s] = reinterpret_cast<const float4*>(xs + s * stream_stride + src * width)[i];
        if (mix) {
            float4* y4 = reinterpret_cast<float4*>(y + src * width);
            const float4 yv = y4[i];
            float4 nv[SN];
#pragma unroll
            for (int t = 0; t < SN; ++t) {
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int s = 0; s < SN; ++s) {
                    const float m = tb.mix[s][t];
                    acc.x = fmaf(m, v[s].x, acc.x); acc.y = fmaf(m, v[s].y, acc.y);
                    acc.z = fmaf(m, v[s].z, acc.z); acc.w = fmaf(m, v[s].w, acc.w);
                }
                const float bt = tb.b[t];
                nv[t] = make_float4(fmaf(bt, yv.x, acc.x), fmaf(bt, yv.y, acc.y), fmaf(bt, yv.z, acc.z), fmaf(bt, yv.w, acc.w));
            }
#pragma unroll
            for (int t = 0; t < SN; ++t) {
                v[t] = nv[t];
                reinterpret_cast<float4*>(xs + t * stream_stride + src * width)[i] = nv[t];
            }
            y4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (do_read) {
            float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int s = 0; s < SN; ++s) {
                const float as = tb.a[s];
                u.x = fmaf(as, v[s].x, u.x); u.y = fmaf(as, v[s].y, u.y); u.z = fmaf(as, v[s].z, u.z); u.w = fmaf(as, v[s].w, u.w);
            }
            u_row4[i] = u;
            ss += u.x * u.x; ss += u.y * u.y; ss += u.z * u.z; ss += u.w * u.w;
        }
    }
    if (!do_read) return;
    ss = block_sum(ss, red);
    const float inv = w ? inv_rms(ss, (float)width, eps) : 1.0f;
    for (int i = threadIdx.x; i < w4; i += blockDim.x) {
        float4 u = u_row4[i];
        if (w) {
            const float4 wv = reinterpret_cast<const float4*>(w)[i];
            u = make_float4(u.x * wv.x * inv, u.y * wv.y * inv, u.z * wv.z * inv, u.w * wv.w * inv);
        }
        TO* o = out + r * width + 4 * i;
        if constexpr (sizeof(TO) == 4) {
            *reinterpret_cast<float4*>(o) = u;
        } else {
            const __nv_bfloat162 lo = __floats2bfloat162_rn(u.x, u.y), hi = __floats2bfloat162_rn(u.z, u.w);
            uint2 pk;
            pk.x = *reinterpret_cast<const unsigned*>(&lo);
            pk.y = *reinterpret_cast<const unsigned*>(&hi);
            *reinterpret_cast<uint2*>(o) = pk;
        }
    }
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
    // four columns a thread where the rows are 16-byte aligned and the number of copies is one the kernel is built for
    const bool vec = width % 4 == 0 && S <= 4 && stream_stride % 4 == 0 && ((uintptr_t)xs & 15) == 0 &&
                     (!y || ((uintptr_t)y & 15) == 0) && (!w || ((uintptr_t)w & 15) == 0) &&
                     (!out || ((uintptr_t)out & 15) == 0);
    if (vec) {
        const int vthreads = width >= 2048 ? 512 : (width >= 1024 ? 256 : 128);
#define GOV(TO, SN) do { \
        if (smem > 48 * 1024) cudaFuncSetAttribute(streams_pass_vec_kernel<TO, SN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        e = ub_launch_dependent(streams_pass_vec_kernel<TO, SN>, dim3(n_rows), dim3(vthreads), smem, st, xs, stream_stride, mix, b, y, a, \
                                do_read, w, rows, (TO*)out, width, eps); } while (0)
#define GOS(TO) do { switch (S) { case 1: GOV(TO, 1); break; case 2: GOV(TO, 2); break; case 3: GOV(TO, 3); break; default: GOV(TO, 4); } } while (0)
        if (out_dtype == UB_F32) GOS(float);
        else if (out_dtype == UB_BF16) GOS(__nv_bfloat16);
        else return UB_ERR_UNSUPPORTED;
#undef GOS
#undef GOV
        return (int)e;
    }
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
