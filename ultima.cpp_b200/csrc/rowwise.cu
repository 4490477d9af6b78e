// Row-wise kernels around a residual stream whose sublayers are scaled channel by channel and read their
// input through a short convolution over time.
//
//   layernorm        (x - mean) / sqrt(var + eps) * w, the variance about the mean, no bias; float32 sums
//   scale_add_norm   x += s * y (s one number a channel), y cleared, and in the same pass the next sublayer's
//                    input: nothing, x in the activation type, an RMS norm or a layer norm of the new x
//   causal_conv      y_t = sum_j w[:, j] u_(t - taps + 1 + j) for every channel of a projection row (the sum of K
//                    slices, plus an optional bias), the inputs of before the step read from per-sequence state,
//                    zeros before a sequence's start; optionally u_t + y_t, a bias of its own, SiLU; optionally a column
//                    range blended with another layer's values of the same token (or handed out for that)
//   causal_conv_state   the last taps - 1 inputs of (state ++ step) become the state (in a step of one token a sequence a
//                    channel's state has one reader, the thread that convolves it, which then moves it on itself)
//   take_cols        a column range of a projection row (summed over its K slices), optionally through tanh,
//                    into the activation type, padded with zeros to an aligned width
//   unary            the exact (erf) GELU or the square of the rectifier, element by element
//   side_gate        gelu_tanh(s) * table[token, column range]
// Sums, norms, the convolution and the activations are float32 whatever the types of input and output.
#include "common.cuh"

constexpr int RW_MAX_TAPS = 16;

__device__ __forceinline__ float rw_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

// ---------------------------------------------------------------------------------------
template <typename TO>
__global__ void layernorm_kernel(const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out,
                                 const int* __restrict__ rows, int width, float eps) {
    __shared__ float red[33];
    pdl_trigger();
    pdl_wait();
    const long long r = rows ? rows[blockIdx.x] : blockIdx.x;
    const float* xr = x + r * width;
    float s = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) s += xr[i];
    const float mean = block_sum(s, red) / (float)width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) { const float d = xr[i] - mean; ss += d * d; }
    const float inv = inv_rms(block_sum(ss, red), (float)width, eps);
    TO* o = out + (long long)blockIdx.x * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_f32<TO>((xr[i] - mean) * inv * w[i]);
}

// The same with a row held in registers: four neighbouring columns a load, one pass over global memory (rows of a
// multiple of 4 columns, up to 256 * 4 * NCH of them).
template <typename TO, int NCH>
__global__ void __launch_bounds__(256)
layernorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out,
                     const int* __restrict__ rows, int width, float eps) {
    __shared__ float red[33];
    pdl_trigger();
    pdl_wait();
    const long long r = rows ? rows[blockIdx.x] : blockIdx.x;
    const float4* xr = reinterpret_cast<const float4*>(x + r * width);
    const int chunks = width >> 2;
    float4 v[NCH];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        const int c = threadIdx.x + i * 256;
        v[i] = c < chunks ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    const float mean = block_sum(s, red) / (float)width;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        if (threadIdx.x + i * 256 < chunks) {
            v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
            ss += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
        }
    }
    const float inv = inv_rms(block_sum(ss, red), (float)width, eps);
    TO* o = out + (long long)blockIdx.x * width;
    const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        const int c = threadIdx.x + i * 256;
        if (c < chunks) {
            const float4 ww = w4[c];
            const float y[4] = {v[i].x * inv * ww.x, v[i].y * inv * ww.y, v[i].z * inv * ww.z, v[i].w * inv * ww.w};
            store_vec<TO, 4>(o + 4 * c, y);
        }
    }
}

UB_API int ub_layernorm(const float* x, const float* w, void* out, int out_dtype, const int* rows, int n_rows, int width,
                        float eps, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    if (width <= 0) return UB_ERR_ARG;
    if (out_dtype != UB_F32 && out_dtype != UB_BF16) return UB_ERR_UNSUPPORTED;
    cudaError_t e;
    const bool aligned = (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
    if (width % 4 == 0 && width <= 256 * 4 * 8 && aligned) {
        const int nch = (width / 4 + 255) / 256;
#define GO(NCH) e = out_dtype == UB_F32 \
            ? ub_launch_dependent(layernorm_vec_kernel<float, NCH>, dim3(n_rows), dim3(256), 0, st, x, w, (float*)out, rows, width, eps) \
            : ub_launch_dependent(layernorm_vec_kernel<__nv_bfloat16, NCH>, dim3(n_rows), dim3(256), 0, st, x, w, (__nv_bfloat16*)out, rows, width, eps)
        if (nch <= 1) GO(1); else if (nch <= 2) GO(2); else if (nch <= 4) GO(4); else GO(8);
#undef GO
        return (int)e;
    }
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    if (out_dtype == UB_F32)
        e = ub_launch_dependent(layernorm_kernel<float>, dim3(n_rows), dim3(threads), 0, st, x, w, (float*)out, rows, width, eps);
    else
        e = ub_launch_dependent(layernorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, st, x, w, (__nv_bfloat16*)out, rows, width, eps);
    return (int)e;
}

// ---------------------------------------------------------------------------------------
// mode: 0 nothing goes out, 1 the new x as it is, 2 its RMS norm times nw, 3 its layer norm times nw
template <typename TO>
__global__ void scale_add_norm_kernel(float* __restrict__ y, const float* __restrict__ scale, float* __restrict__ x, int mode,
                                      const float* __restrict__ nw, float eps, TO* __restrict__ out, int width, int clear_y) {
    __shared__ float red[33];
    pdl_trigger();
    pdl_wait();
    const long long r = blockIdx.x;
    float* yr = y + r * width;
    float* xr = x + r * width;
    float s = 0.f, ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = fmaf(yr[i], scale ? scale[i] : 1.0f, xr[i]);
        xr[i] = v;
        if (clear_y) yr[i] = 0.f;
        s += v;
        ss += v * v;
    }
    if (mode == 0) return;
    TO* o = out + r * width;
    if (mode == 1) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_f32<TO>(xr[i]);      // (this thread's own writes)
        return;
    }
    float mean = 0.f;
    if (mode == 3) {
        mean = block_sum(s, red) / (float)width;
        ss = 0.f;
        for (int i = threadIdx.x; i < width; i += blockDim.x) { const float d = xr[i] - mean; ss += d * d; }
    }
    const float inv = inv_rms(block_sum(ss, red), (float)width, eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_f32<TO>((xr[i] - mean) * inv * nw[i]);
}

UB_API int ub_scale_add_norm(float* y, const float* scale, float* x, int mode, const float* nw, float eps, void* out,
                             int out_dtype, int n_rows, int width, int clear_y, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    if (width <= 0 || mode < 0 || mode > 3 || (mode >= 2 && !nw) || (mode >= 1 && !out)) return UB_ERR_ARG;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    cudaError_t e;
    if (mode == 0 || out_dtype == UB_F32)
        e = ub_launch_dependent(scale_add_norm_kernel<float>, dim3(n_rows), dim3(threads), 0, st, y, scale, x, mode, nw, eps, (float*)out, width, clear_y);
    else if (out_dtype == UB_BF16)
        e = ub_launch_dependent(scale_add_norm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, st, y, scale, x, mode, nw, eps, (__nv_bfloat16*)out, width, clear_y);
    else return UB_ERR_UNSUPPORTED;
    return (int)e;
}

// ---------------------------------------------------------------------------------------
struct ConvIn {
    const void* x;           // [parts][T][ldx], the channels from column col_off on
    long long ldx, part_stride;
    int n_parts, col_off;
    const float* bias;       // [C] or null: added to every input (the state holds inputs with it)
};

template <typename TX>
__device__ __forceinline__ float conv_input(const ConvIn& in, long long t, int c) {
    const TX* x = (const TX*)in.x;
    float v = 0.f;
    for (int p = 0; p < in.n_parts; ++p) v += to_f32<TX>(x[p * in.part_stride + t * in.ldx + in.col_off + c]);
    return in.bias ? v + in.bias[c] : v;
}

// One thread a (token, channel).  mix_mode 1: the channels [mix_lo, mix_hi) go out to ``shared`` as they are (another
// layer blends them into its own); 2: they become (1 - lam) * own + lam * shared[t].
template <typename TX, typename TO>
__global__ void __launch_bounds__(256)
causal_conv_kernel(ConvIn in, const float* __restrict__ w, float* __restrict__ state, int update_state, const int* __restrict__ tok_seq,
                   const int* __restrict__ seq_start, const int* __restrict__ seq_slot, TO* __restrict__ out, long long ldo,
                   int n_tokens, int C, int taps, int add_input, int act, int mix_mode, int mix_lo, int mix_hi,
                   const float* __restrict__ lam, float* __restrict__ shared, const float* __restrict__ out_bias) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const long long t = blockIdx.x;
    if (c >= C) return;
    const float u = conv_input<TX>(in, t, c);
    float acc = u;
    if (taps > 0) {
        const int seq = tok_seq[t];
        const int r = (int)t - seq_start[seq];
        const int K = taps - 1;
        float* st = state + (long long)seq_slot[seq] * K * C;
        acc = 0.f;
        for (int j = K; j >= 1; --j) {                 // oldest input first
            const float xv = (r - j >= 0) ? conv_input<TX>(in, t - j, c) : st[(long long)(K + r - j) * C + c];
            acc = fmaf(w[(long long)c * taps + (K - j)], xv, acc);
            if (update_state && j < K) st[(long long)(K - 1 - j) * C + c] = xv;      // r = 0: the input j back becomes j + 1 back
        }
        if (update_state && K > 0) st[(long long)(K - 1) * C + c] = u;
        acc = fmaf(w[(long long)c * taps + K], u, acc);
        if (add_input) acc += u;
    }
    if (out_bias) acc += out_bias[c];                  // a bias of the convolution itself (the state holds inputs without it)
    if (act == 1) acc *= rw_sigmoid(acc);
    if (mix_mode && c >= mix_lo && c < mix_hi) {
        float* sh = shared + t * (mix_hi - mix_lo) + (c - mix_lo);
        if (mix_mode == 1) *sh = acc;
        else { const float l = *lam; acc = (1.0f - l) * acc + l * *sh; }
    }
    out[t * ldo + c] = from_f32<TO>(acc);
}

// The same for 2 to 4 taps with a thread walking CONV_TILE tokens of its channel in a row: an input is read once and kept
// for the tokens behind it.  The first K tokens of a tile, and a sequence's first K tokens of the step, take their
// earlier inputs the long way (rows of the step, or the state).
constexpr int CONV_TILE = 16;

template <typename TX, typename TO, int K>
__global__ void __launch_bounds__(256)
causal_conv_tile_kernel(ConvIn in, const float* __restrict__ w, float* __restrict__ state, int update_state,
                        const int* __restrict__ tok_seq, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                        TO* __restrict__ out, long long ldo, int n_tokens, int C, int add_input, int act, int mix_mode, int mix_lo,
                        int mix_hi, const float* __restrict__ lam, float* __restrict__ shared, const float* __restrict__ out_bias) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float wt[K + 1], win[K];                           // win[j - 1]: the input j tokens back
#pragma unroll
    for (int j = 0; j <= K; ++j) wt[j] = w[(long long)c * (K + 1) + j];
#pragma unroll
    for (int j = 0; j < K; ++j) win[j] = 0.f;
    const float ob = out_bias ? out_bias[c] : 0.f;
    const bool mixes = mix_mode && c >= mix_lo && c < mix_hi;
    const float l = (mixes && mix_mode == 2) ? *lam : 0.f;
    const long long tbase = (long long)blockIdx.x * CONV_TILE;
    // the tile's sequence once where the whole tile lies in one (tokens of a sequence stand together, so the first and the
    // last token tell); a token's input is asked for while the token before it is worked on
    const int seq0 = tok_seq[tbase];
    const bool one_seq = tok_seq[min(tbase + CONV_TILE - 1, (long long)n_tokens - 1)] == seq0;
    const int r0 = (int)tbase - seq_start[seq0];
    float u_next = conv_input<TX>(in, tbase, c);
    for (int i = 0; i < CONV_TILE; ++i) {
        const long long t = tbase + i;
        if (t >= n_tokens) break;
        const float u = u_next;
        if (i + 1 < CONV_TILE && t + 1 < n_tokens) u_next = conv_input<TX>(in, t + 1, c);
        const int seq = one_seq ? seq0 : tok_seq[t];
        const int r = one_seq ? r0 + i : (int)t - seq_start[seq];
        float acc = 0.f;
        if (i >= K && r >= K) {
#pragma unroll
            for (int j = K; j >= 1; --j) acc = fmaf(wt[K - j], win[j - 1], acc);
        } else {
            float* st = state + (long long)seq_slot[seq] * K * C;
#pragma unroll
            for (int j = K; j >= 1; --j) {
                const float xv = (r - j >= 0) ? conv_input<TX>(in, t - j, c) : st[(long long)(K + r - j) * C + c];
                acc = fmaf(wt[K - j], xv, acc);
                if (update_state && j < K) st[(long long)(K - 1 - j) * C + c] = xv;
            }
            if (update_state) st[(long long)(K - 1) * C + c] = u;
        }
        acc = fmaf(wt[K], u, acc);
        if (add_input) acc += u;
        acc += ob;
        if (act == 1) acc *= rw_sigmoid(acc);
        if (mixes) {
            float* sh = shared + t * (mix_hi - mix_lo) + (c - mix_lo);
            if (mix_mode == 1) *sh = acc;
            else acc = (1.0f - l) * acc + l * *sh;
        }
        out[t * ldo + c] = from_f32<TO>(acc);
#pragma unroll
        for (int j = K - 1; j >= 1; --j) win[j] = win[j - 1];
        win[0] = u;
    }
}

// The tile walk with four neighbouring channels a thread (16-byte loads of float32, 8-byte loads of bfloat16): rows, column
// ranges and the state on 16-byte boundaries, channels a multiple of 4.
template <typename TX>
__device__ __forceinline__ float4 conv_input4(const ConvIn& in, long long t, int c) {
    const TX* x = (const TX*)in.x;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    for (int p = 0; p < in.n_parts; ++p) {
        float a[4];
        load_vec<TX, 4>(x + p * in.part_stride + t * in.ldx + in.col_off + c, a);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] += a[e];
    }
    if (in.bias) {
        const float4 b = *reinterpret_cast<const float4*>(in.bias + c);
        v[0] += b.x; v[1] += b.y; v[2] += b.z; v[3] += b.w;
    }
    return make_float4(v[0], v[1], v[2], v[3]);
}

__device__ __forceinline__ void fma4(float4& acc, const float* w, const float4& x) {
    acc.x = fmaf(w[0], x.x, acc.x); acc.y = fmaf(w[1], x.y, acc.y); acc.z = fmaf(w[2], x.z, acc.z); acc.w = fmaf(w[3], x.w, acc.w);
}

template <typename TX, typename TO, int K>
__global__ void __launch_bounds__(128)
causal_conv_vec4_kernel(ConvIn in, const float* __restrict__ w, const float* __restrict__ state,
                        const int* __restrict__ tok_seq, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                        TO* __restrict__ out, long long ldo, int n_tokens, int C, int add_input, int act, int mix_mode, int mix_lo,
                        int mix_hi, const float* __restrict__ lam, float* __restrict__ shared, const float* __restrict__ out_bias) {
    pdl_trigger();
    pdl_wait();
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (c >= C) return;
    float wt[K + 1][4];
#pragma unroll
    for (int j = 0; j <= K; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) wt[j][e] = w[(long long)(c + e) * (K + 1) + j];
    float4 win[K];
#pragma unroll
    for (int j = 0; j < K; ++j) win[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 ob = out_bias ? *reinterpret_cast<const float4*>(out_bias + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    const bool mixes = mix_mode && c >= mix_lo && c < mix_hi;
    const float l = (mixes && mix_mode == 2) ? *lam : 0.f;
    const long long tbase = (long long)blockIdx.x * CONV_TILE;
    const int seq0 = tok_seq[tbase];
    const bool one_seq = tok_seq[min(tbase + CONV_TILE - 1, (long long)n_tokens - 1)] == seq0;
    const int r0 = (int)tbase - seq_start[seq0];
    float4 u_next = conv_input4<TX>(in, tbase, c);
    for (int i = 0; i < CONV_TILE; ++i) {
        const long long t = tbase + i;
        if (t >= n_tokens) break;
        const float4 u = u_next;
        if (i + 1 < CONV_TILE && t + 1 < n_tokens) u_next = conv_input4<TX>(in, t + 1, c);
        const int seq = one_seq ? seq0 : tok_seq[t];
        const int r = one_seq ? r0 + i : (int)t - seq_start[seq];
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i >= K && r >= K) {
#pragma unroll
            for (int j = K; j >= 1; --j) fma4(acc, wt[K - j], win[j - 1]);
        } else {
            const float* st = state + (long long)seq_slot[seq] * K * C;
#pragma unroll
            for (int j = K; j >= 1; --j) {
                const float4 xv = (r - j >= 0) ? conv_input4<TX>(in, t - j, c)
                                               : *reinterpret_cast<const float4*>(st + (long long)(K + r - j) * C + c);
                fma4(acc, wt[K - j], xv);
            }
        }
        fma4(acc, wt[K], u);
        float y[4] = {acc.x, acc.y, acc.z, acc.w};
        const float uu[4] = {u.x, u.y, u.z, u.w}, obv[4] = {ob.x, ob.y, ob.z, ob.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (add_input) y[e] += uu[e];
            y[e] += obv[e];
            if (act == 1) y[e] *= rw_sigmoid(y[e]);
        }
        if (mixes) {
            float4* sh = reinterpret_cast<float4*>(shared + t * (mix_hi - mix_lo) + (c - mix_lo));
            if (mix_mode == 1) *sh = make_float4(y[0], y[1], y[2], y[3]);
            else {
                const float4 o = *sh;
                y[0] = (1.0f - l) * y[0] + l * o.x; y[1] = (1.0f - l) * y[1] + l * o.y;
                y[2] = (1.0f - l) * y[2] + l * o.z; y[3] = (1.0f - l) * y[3] + l * o.w;
            }
        }
        store_vec<TO, 4>(out + t * ldo + c, y);
#pragma unroll
        for (int j = K - 1; j >= 1; --j) win[j] = win[j - 1];
        win[0] = u;
    }
}

// One thread a (sequence, channel).
template <typename TX>
__global__ void causal_conv_state_kernel(ConvIn in, float* __restrict__ state, const int* __restrict__ seq_start,
                                         const int* __restrict__ seq_slot, int n_seqs, int C, int taps) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_seqs * C) return;
    const int b = (int)(i / C), c = (int)(i % C);
    const int K = taps - 1;
    const int first = seq_start[b], n = seq_start[b + 1] - first;
    float* st = state + (long long)seq_slot[b] * K * C;
    float tmp[RW_MAX_TAPS];
    for (int k = 0; k < K; ++k) {
        const int rel = n - K + k;
        tmp[k] = rel >= 0 ? conv_input<TX>(in, first + rel, c) : st[(long long)(K + rel) * C + c];
    }
    for (int k = 0; k < K; ++k) st[(long long)k * C + c] = tmp[k];
}

UB_API int ub_causal_conv(const void* x, int x_dtype, long long ldx, int n_parts, long long part_stride, int col_off,
                          const float* bias, const float* w, float* state, int update_state, const int* tok_seq, const int* seq_start,
                          const int* seq_slot, void* out, int out_dtype, long long ldo, int n_tokens, int C, int taps,
                          int add_input, int act, int mix_mode, int mix_lo, int mix_hi, const float* lam, float* shared,
                          const float* out_bias, cudaStream_t st) {
    if (n_tokens <= 0 || C <= 0) return 0;
    if (taps < 0 || taps > RW_MAX_TAPS || n_parts < 1 || (taps > 1 && !state) || (taps > 0 && !w)) return UB_ERR_ARG;
    if (mix_mode && (!shared || mix_lo < 0 || mix_hi > C || mix_lo >= mix_hi || (mix_mode == 2 && !lam))) return UB_ERR_ARG;
    ConvIn in = {x, ldx, part_stride, n_parts, col_off, bias};
    if (update_state && taps < 2) update_state = 0;
    const dim3 grid(n_tokens, (C + 255) / 256), block(256);
    const dim3 tgrid((n_tokens + CONV_TILE - 1) / CONV_TILE, (C + 255) / 256);
    // few tokens, or one a sequence: a thread a (token, channel), since a walk over tokens that all take the long way is slow
    const bool tiled = !update_state && n_tokens >= 4 * CONV_TILE;
    cudaError_t e;
#define ARGS(TO) in, w, state, update_state, tok_seq, seq_start, seq_slot, (TO*)out, ldo, n_tokens, C
#define TAIL add_input, act, mix_mode, mix_lo, mix_hi, lam, shared, out_bias
    // four channels a thread where everything lies on 16-byte boundaries
    const size_t xe = x_dtype == UB_F32 ? 4 : 2, oe = out_dtype == UB_F32 ? 4 : 2;
    const bool vec4 = tiled && taps >= 2 && taps <= 4 && C % 4 == 0 && col_off % 4 == 0 && ldx % 4 == 0 && part_stride % 4 == 0 &&
        ldo % 4 == 0 && ((uintptr_t)x % (4 * xe)) == 0 && ((uintptr_t)out % (4 * oe)) == 0 &&
        (((uintptr_t)bias | (uintptr_t)out_bias | (uintptr_t)state | (uintptr_t)shared) & 15) == 0 &&
        (!mix_mode || (mix_lo % 4 == 0 && mix_hi % 4 == 0));
    const dim3 vgrid((n_tokens + CONV_TILE - 1) / CONV_TILE, (C / 4 + 127) / 128), vblock(128);
#define VARGS(TO) in, w, (const float*)state, tok_seq, seq_start, seq_slot, (TO*)out, ldo, n_tokens, C
#define GO(TX, TO) do { \
        if (vec4 && taps == 2) e = ub_launch_dependent(causal_conv_vec4_kernel<TX, TO, 1>, vgrid, vblock, 0, st, VARGS(TO), TAIL); \
        else if (vec4 && taps == 3) e = ub_launch_dependent(causal_conv_vec4_kernel<TX, TO, 2>, vgrid, vblock, 0, st, VARGS(TO), TAIL); \
        else if (vec4) e = ub_launch_dependent(causal_conv_vec4_kernel<TX, TO, 3>, vgrid, vblock, 0, st, VARGS(TO), TAIL); \
        else if (!tiled) e = ub_launch_dependent(causal_conv_kernel<TX, TO>, grid, block, 0, st, ARGS(TO), taps, TAIL); \
        else if (taps == 2) e = ub_launch_dependent(causal_conv_tile_kernel<TX, TO, 1>, tgrid, block, 0, st, ARGS(TO), TAIL); \
        else if (taps == 3) e = ub_launch_dependent(causal_conv_tile_kernel<TX, TO, 2>, tgrid, block, 0, st, ARGS(TO), TAIL); \
        else if (taps == 4) e = ub_launch_dependent(causal_conv_tile_kernel<TX, TO, 3>, tgrid, block, 0, st, ARGS(TO), TAIL); \
        else e = ub_launch_dependent(causal_conv_kernel<TX, TO>, grid, block, 0, st, ARGS(TO), taps, TAIL); } while (0)
    if (x_dtype == UB_F32 && out_dtype == UB_F32) GO(float, float);
    else if (x_dtype == UB_F32 && out_dtype == UB_BF16) GO(float, __nv_bfloat16);
    else if (x_dtype == UB_BF16 && out_dtype == UB_BF16) GO(__nv_bfloat16, __nv_bfloat16);
    else return UB_ERR_UNSUPPORTED;
#undef GO
#undef ARGS
#undef VARGS
#undef TAIL
    return (int)e;
}

UB_API int ub_causal_conv_state(const void* x, int x_dtype, long long ldx, int n_parts, long long part_stride, int col_off,
                                const float* bias, float* state, const int* seq_start, const int* seq_slot, int n_seqs, int C,
                                int taps, cudaStream_t st) {
    if (n_seqs <= 0 || taps <= 1 || C <= 0) return 0;
    if (taps > RW_MAX_TAPS || n_parts < 1) return UB_ERR_ARG;
    ConvIn in = {x, ldx, part_stride, n_parts, col_off, bias};
    const long long n = (long long)n_seqs * C;
    const dim3 grid((unsigned)((n + 127) / 128)), block(128);
    cudaError_t e;
    if (x_dtype == UB_F32) e = ub_launch_dependent(causal_conv_state_kernel<float>, grid, block, 0, st, in, state, seq_start, seq_slot, n_seqs, C, taps);
    else if (x_dtype == UB_BF16) e = ub_launch_dependent(causal_conv_state_kernel<__nv_bfloat16>, grid, block, 0, st, in, state, seq_start, seq_slot, n_seqs, C, taps);
    else return UB_ERR_UNSUPPORTED;
    return (int)e;
}

// ---------------------------------------------------------------------------------------
template <typename TO>
__global__ void take_cols_kernel(const float* __restrict__ x, long long ldx, int n_parts, long long part_stride, int col_off,
                                 int n, int act, TO* __restrict__ out, long long ldo, int n_out, long long total) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / n_out;
    const int j = (int)(i % n_out);
    float v = 0.f;
    if (j < n) {
        for (int p = 0; p < n_parts; ++p) v += x[p * part_stride + t * ldx + col_off + j];
        if (act == 1) v = tanhf(v);
    }
    out[t * ldo + j] = from_f32<TO>(v);
}

UB_API int ub_take_cols(const float* x, long long ldx, int n_parts, long long part_stride, int col_off, int n, int act, void* out,
                        int out_dtype, long long ldo, int n_out, int n_tokens, cudaStream_t st) {
    const long long total = (long long)n_tokens * n_out;
    if (total <= 0) return 0;
    if (n_parts < 1 || n > n_out) return UB_ERR_ARG;
    const dim3 grid((unsigned)((total + 255) / 256)), block(256);
    cudaError_t e;
    if (out_dtype == UB_F32) e = ub_launch_dependent(take_cols_kernel<float>, grid, block, 0, st, x, ldx, n_parts, part_stride, col_off, n, act, (float*)out, ldo, n_out, total);
    else if (out_dtype == UB_BF16) e = ub_launch_dependent(take_cols_kernel<__nv_bfloat16>, grid, block, 0, st, x, ldx, n_parts, part_stride, col_off, n, act, (__nv_bfloat16*)out, ldo, n_out, total);
    else return UB_ERR_UNSUPPORTED;
    return (int)e;
}

// ---------------------------------------------------------------------------------------
// kind 1: 0.5 z (1 + erf(z / sqrt 2)); 2: max(z, 0)^2
template <typename TI, typename TO>
__global__ void unary_kernel(const TI* __restrict__ in, TO* __restrict__ out, long long n, int kind) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float z = to_f32<TI>(in[i]);
    float v;
    if (kind == 1) v = 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
    else { const float p = fmaxf(z, 0.f); v = p * p; }
    out[i] = from_f32<TO>(v);
}

UB_API int ub_unary(const void* in, int in_dtype, void* out, int out_dtype, long long n, int kind, cudaStream_t st) {
    if (n <= 0) return 0;
    if (kind != 1 && kind != 2) return UB_ERR_ARG;
    const dim3 grid((unsigned)((n + 255) / 256)), block(256);
    cudaError_t e;
#define GO(TI, TO) e = ub_launch_dependent(unary_kernel<TI, TO>, grid, block, 0, st, (const TI*)in, (TO*)out, n, kind)
    if (in_dtype == UB_F32 && out_dtype == UB_F32) GO(float, float);
    else if (in_dtype == UB_F32 && out_dtype == UB_BF16) GO(float, __nv_bfloat16);
    else if (in_dtype == UB_BF16 && out_dtype == UB_BF16) GO(__nv_bfloat16, __nv_bfloat16);
    else return UB_ERR_UNSUPPORTED;
#undef GO
    return (int)e;
}

// ---------------------------------------------------------------------------------------
// out[t, j] = gelu_tanh(s[t, j]) * table[ids[t], col0 + j] for j < dim, zero up to n_out
template <typename TT, typename TO>
__global__ void side_gate_kernel(const float* __restrict__ s, long long lds, const TT* __restrict__ table, long long ldt, int col0,
                                 const int* __restrict__ ids, int vocab, TO* __restrict__ out, long long ldo, int dim, int n_out,
                                 long long total) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / n_out;
    const int j = (int)(i % n_out);
    float v = 0.f;
    const int id = ids[t];
    if (j < dim && id >= 0 && id < vocab) {
        const float z = s[t * lds + j];
        const float g = 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
        v = g * to_f32<TT>(table[(long long)id * ldt + col0 + j]);
    }
    out[t * ldo + j] = from_f32<TO>(v);
}

UB_API int ub_side_gate(const float* s, long long lds, const void* table, int table_dtype, long long ldt, int col0, const int* ids,
                        int vocab, void* out, int out_dtype, long long ldo, int dim, int n_out, int n_tokens, cudaStream_t st) {
    const long long total = (long long)n_tokens * n_out;
    if (total <= 0) return 0;
    if (dim > n_out) return UB_ERR_ARG;
    const dim3 grid((unsigned)((total + 255) / 256)), block(256);
    cudaError_t e;
#define GO(TT, TO) e = ub_launch_dependent(side_gate_kernel<TT, TO>, grid, block, 0, st, s, lds, (const TT*)table, ldt, col0, ids, vocab, \
                                           (TO*)out, ldo, dim, n_out, total)
    if (table_dtype == UB_F32 && out_dtype == UB_F32) GO(float, float);
    else if (table_dtype == UB_BF16 && out_dtype == UB_BF16) GO(__nv_bfloat16, __nv_bfloat16);
    else if (table_dtype == UB_F32 && out_dtype == UB_BF16) GO(float, __nv_bfloat16);
    else return UB_ERR_UNSUPPORTED;
#undef GO
    return (int)e;
}
