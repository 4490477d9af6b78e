// A selective state-space mixer with a scalar decay a head (the "state-space duality" form): for every
// head a matrix S [N, P] (N state channels, P value channels) in float32, zero at a sequence's start, plus
// the last inputs of a short causal convolution.  For one token of one head, with a step size dt > 0,
// an input row B [N] and an output row C [N] (shared by the heads of a group) and the value x [P]:
//     S <- exp(-exp(A_log) dt) S + dt B x^T;      y = S^T C + D x
//
// A projection row is laid out [z | x | B | C | dt]: the output gate, then the convolution's channels
// (x, B, C), then one step size a head.  Four kernels, for prompts and single tokens alike (a step's
// tokens of one sequence are rows seq_start[s] .. seq_start[s + 1] of the packed batch; state rows are
// slot numbers):
//   ssm_prepare            convolution + bias + SiLU of x, B, C; dt = softplus(. + dt_bias); the decay
//   ssm_conv_state_update  the convolution's last inputs, carried to the next step
//   ssm_scan               the recurrence
//   ssm_finish             y silu(z), RMS norm in equal parts of the row, weight, output scale
// Everything is float32; the projection comes in as float32 sums of the product (for few tokens as the
// partial sums of K slices, which the kernels add up as they read).  Every column of S evolves on its
// own and tokens are taken in order, so no sum depends on the batch or on how a prompt was cut.
#include "common.cuh"

constexpr int SSM_MAX_TAPS = 16;

struct SsmShape {
    int H, P, N, G;          // heads, value size, state size, groups of heads that share B and C
    int taps;                // convolution length (the last tap is the current token's)
    int z_off, x_off, b_off, c_off, dt_off;   // columns of a projection row; x, B, C follow one another
    long long ldp;           // row stride of the projection
    int n_parts;             // the projection row is the sum of this many partial results ...
    long long part_stride;   // ... this many elements apart
};

__device__ __forceinline__ float ssm_proj(const float* __restrict__ p, const SsmShape& s, long long t, int c) {
    float v = 0.f;
    for (int i = 0; i < s.n_parts; ++i) v += p[i * s.part_stride + t * s.ldp + c];
    return v;
}
__device__ __forceinline__ float ssm_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// One thread a (token, channel): the convolution's channels first, then one (dt, decay) a head.
// ``update_state`` (only when every sequence brings ONE token, so that a channel's state has this thread
// as its only reader): the convolution's state moves on here.
__global__ void __launch_bounds__(256)
ssm_prepare_kernel(const float* __restrict__ p, SsmShape s, const float* __restrict__ conv_w, const float* __restrict__ conv_b,
                   float* conv_state, int update_state, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                   const int* __restrict__ tok_seq, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                   float* __restrict__ xbc, float* __restrict__ dtv, float* __restrict__ dec, int n_tokens) {
    pdl_trigger();
    pdl_wait();
    const int C = s.H * s.P + 2 * s.G * s.N;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_tokens * (C + s.H)) return;
    const int t = (int)(i / (C + s.H)), c = (int)(i % (C + s.H));
    if (c >= C) {
        const int h = c - C;
        const float dt = ssm_softplus(ssm_proj(p, s, t, s.dt_off + h) + dt_bias[h]);
        dtv[(long long)t * s.H + h] = dt;
        dec[(long long)t * s.H + h] = expf(-expf(a_log[h]) * dt);
        return;
    }
    const int seq = tok_seq[t];
    const int r = t - seq_start[seq];
    const int K = s.taps - 1;
    float* st = conv_state + (long long)seq_slot[seq] * K * C;
    float acc = conv_b ? conv_b[c] : 0.f;
    for (int j = K; j >= 0; --j) {                     // oldest input first
        const float w = conv_w[(long long)c * s.taps + (K - j)];
        const float x = (r - j >= 0) ? ssm_proj(p, s, t - j, s.x_off + c) : st[(long long)(K + r - j) * C + c];
        acc = fmaf(w, x, acc);
        if (update_state && j < K) st[(long long)(K - 1 - j) * C + c] = x;     // r = 0: the input j back becomes j + 1 back
    }
    xbc[(long long)t * C + c] = acc / (1.0f + expf(-acc));
}

// One thread a (sequence, channel): the last taps - 1 inputs of what the state held followed by the step's.
__global__ void ssm_conv_state_update_kernel(const float* __restrict__ p, SsmShape s, float* __restrict__ conv_state,
                                             const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                                             int n_seqs) {
    pdl_trigger();
    pdl_wait();
    const int C = s.H * s.P + 2 * s.G * s.N;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_seqs * C) return;
    const int b = (int)(i / C), c = (int)(i % C);
    const int K = s.taps - 1;
    const int first = seq_start[b], n = seq_start[b + 1] - first;
    float* st = conv_state + (long long)seq_slot[b] * K * C;
    float tmp[SSM_MAX_TAPS];
    for (int k = 0; k < K; ++k) {
        const int rel = n - K + k;
        tmp[k] = rel >= 0 ? ssm_proj(p, s, first + rel, s.x_off + c) : st[(long long)(K + rel) * C + c];
    }
    for (int k = 0; k < K; ++k) st[(long long)k * C + c] = tmp[k];
}

// The recurrence.  A block of 256 threads takes 256 / LANES * CPT value channels of one head of one sequence; LANES
// (8, 16 or 32, by the state's size alone, so that the order of every sum is the same whatever the batch) lanes
// hold one column of S, lane l the state channels of the float4 chunks l, l + LANES, ...: the lanes of a column
// read consecutive bytes of shared memory in one instruction.  More lanes a column mean more warps with fewer
// values each: the kernel is bound by the latency of a token's chain, which many warps hide.  A thread holds
// CPT neighbouring columns, which share its reads of B and C (the kernel issues fewer instructions an element).  Tokens come through shared memory a stage at a time,
// the next stage asked for (cp.async) while this one is worked on.  The state's update does not wait for the
// read-out: a token costs two operations a state element and three exchanges.
__device__ __forceinline__ void ssm_cp4(float* dst, const float* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void ssm_cp16(float* dst, const float* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

// Stages of tokens in shared memory: SSM_STAGES - 1 of them are on their way while one is worked on (a copy from
// the L2 takes about as long as the arithmetic of several dozen tokens).
constexpr int SSM_STAGES = 4;
// CPT: columns of S a thread holds (1 or 2): they share every read of B and C.  A column's sums have the same order
// either way, so the choice (by how many blocks a launch has) changes no bit of the result.
template <int R, int LANES, int CPT>
struct SsmScanLayout {
    static constexpr int NP = LANES * R, COLS = 256 / LANES * CPT;
    static constexpr int TT = NP <= 128 ? 16 : 8;         // tokens a stage
    static constexpr size_t BYTES = (size_t)SSM_STAGES * TT * (2 * NP + COLS + 2) * sizeof(float);
};

// VEC: N, P and the row stride are multiples of 4 and xbc starts on a 16-byte boundary: 16-byte copies.
template <int R, int LANES, int CPT, bool VEC>
__global__ void __launch_bounds__(256)
ssm_scan_kernel(const float* __restrict__ xbc, const float* __restrict__ dtv, const float* __restrict__ dec,
                const float* __restrict__ Dw, float* __restrict__ y, float* __restrict__ S,
                const int* __restrict__ seq_start, const int* __restrict__ seq_slot, int H, int P, int N, int G) {
    static_assert(R % 4 == 0, "a lane holds whole float4 chunks");
    constexpr int COLS = 256 / LANES * CPT, NP = LANES * R, NC = R / 4;
    constexpr int TT = SsmScanLayout<R, LANES, CPT>::TT, ST = SSM_STAGES;
    extern __shared__ __align__(16) float smem[];
    float (*sB)[TT][NP] = reinterpret_cast<float (*)[TT][NP]>(smem);                       // [ST][TT][NP]
    float (*sC)[TT][NP] = reinterpret_cast<float (*)[TT][NP]>(smem + ST * TT * NP);
    float (*sx)[TT][COLS] = reinterpret_cast<float (*)[TT][COLS]>(smem + 2 * ST * TT * NP);
    float (*sdt)[TT] = reinterpret_cast<float (*)[TT]>(smem + 2 * ST * TT * NP + ST * TT * COLS);
    float (*sa)[TT] = reinterpret_cast<float (*)[TT]>(smem + 2 * ST * TT * NP + ST * TT * COLS + ST * TT);
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, col = (tid / LANES) * CPT, l = tid % LANES;      // col: the first of this thread's columns
    const int h = blockIdx.y, b = blockIdx.z, g = h / (H / G);
    const int j = blockIdx.x * COLS + col;
    const int t0 = seq_start[b], t1 = seq_start[b + 1];
    if (t0 >= t1) return;
    const int C = H * P + 2 * G * N;
    float* Sh = S + ((long long)seq_slot[b] * H + h) * N * P;
    float s[CPT][R];
#pragma unroll
    for (int c = 0; c < CPT; ++c)
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int n = ((i >> 2) * LANES + l) * 4 + (i & 3);
            s[c][i] = (n < N && j + c < P) ? Sh[(long long)n * P + j + c] : 0.f;
        }
    const float dh = Dw[h];
    if (t1 - t0 == 1) {
        // one token (a decode step): straight from global memory, no stages
        const float* rowp = xbc + (long long)t0 * C;
        const float a = dec[(long long)t0 * H + h];
        const float dt = dtv[(long long)t0 * H + h];
        float xv[CPT], u[CPT], part[CPT][4];
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            xv[c] = j + c < P ? rowp[h * P + j + c] : 0.f;
            u[c] = dt * xv[c];
            part[c][0] = part[c][1] = part[c][2] = part[c][3] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int n = ((i >> 2) * LANES + l) * 4 + (i & 3);
            const float bv = n < N ? rowp[H * P + g * N + n] : 0.f;
            const float cv = n < N ? rowp[H * P + G * N + g * N + n] : 0.f;
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                s[c][i] = fmaf(a, s[c][i], bv * u[c]);
                part[c][i & 3] = fmaf(s[c][i], cv, part[c][i & 3]);
                if (n < N && j + c < P) Sh[(long long)n * P + j + c] = s[c][i];
            }
        }
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            float sum = (part[c][0] + part[c][1]) + (part[c][2] + part[c][3]);   // (the order of the stages' sum: chunk by chunk, then the four)
#pragma unroll
            for (int w = 1; w < LANES; w <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, w);
            if (l == 0 && j + c < P) y[((long long)t0 * H + h) * P + j + c] = fmaf(dh, xv[c], sum);
        }
        return;
    }
    // channels past the sizes are zeros that no copy ever touches
    for (int idx = tid; idx < ST * TT * NP; idx += blockDim.x)
        if (idx % NP >= N) { (&sB[0][0][0])[idx] = 0.f; (&sC[0][0][0])[idx] = 0.f; }
    for (int idx = tid; idx < ST * TT * COLS; idx += blockDim.x)
        if (blockIdx.x * COLS + idx % COLS >= P) (&sx[0][0][0])[idx] = 0.f;
    const float* brow = xbc + H * P + g * N;
    const float* xrow = xbc + h * P + blockIdx.x * COLS;
    // one group of copies is committed for every stage, empty past the end, so the count to wait for is fixed
    auto fetch = [&](int base, int buf) {
        const int cnt = min(TT, t1 - base);
        if (cnt > 0) {
            if (VEC) {
                const int n4 = N >> 2;
                for (int idx = tid; idx < cnt * n4; idx += blockDim.x) {
                    const int tt = idx / n4, n = (idx % n4) * 4;
                    const float* rowp = brow + (long long)(base + tt) * C;
                    ssm_cp16(&sB[buf][tt][n], rowp + n);
                    ssm_cp16(&sC[buf][tt][n], rowp + G * N + n);
                }
                for (int idx = tid; idx < cnt * (COLS / 4); idx += blockDim.x) {
                    const int tt = idx / (COLS / 4), cc = (idx % (COLS / 4)) * 4;
                    if (blockIdx.x * COLS + cc < P) ssm_cp16(&sx[buf][tt][cc], xrow + (long long)(base + tt) * C + cc);
                }
            } else {
                for (int idx = tid; idx < cnt * N; idx += blockDim.x) {
                    const int tt = idx / N, n = idx % N;
                    const float* rowp = brow + (long long)(base + tt) * C;
                    ssm_cp4(&sB[buf][tt][n], rowp + n);
                    ssm_cp4(&sC[buf][tt][n], rowp + G * N + n);
                }
                for (int idx = tid; idx < cnt * COLS; idx += blockDim.x) {
                    const int tt = idx / COLS, cc = idx % COLS;
                    if (blockIdx.x * COLS + cc < P) ssm_cp4(&sx[buf][tt][cc], xrow + (long long)(base + tt) * C + cc);
                }
            }
            if (tid >= 128 && tid < 128 + cnt) ssm_cp4(&sdt[buf][tid - 128], dtv + (long long)(base + tid - 128) * H + h);
            if (tid >= 192 && tid < 192 + cnt) ssm_cp4(&sa[buf][tid - 192], dec + (long long)(base + tid - 192) * H + h);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    __syncthreads();                                       // the constants above are in place before any copy lands beside them
#pragma unroll
    for (int i = 0; i < ST - 1; ++i) fetch(t0 + i * TT, i);
    int buf = 0;
    float* yp = y + ((long long)t0 * H + h) * P + j;       // this thread's place in a token's output row
    const long long ystep = (long long)H * P;
    for (int base = t0; base < t1; base += TT, buf = (buf + 1) % ST) {
        const int cnt = min(TT, t1 - base);
        fetch(base + (ST - 1) * TT, (buf + ST - 1) % ST);  // (that buffer's readers passed the barrier at the end of the last round)
        asm volatile("cp.async.wait_group %0;" ::"n"(ST - 1) : "memory");
        __syncthreads();
        auto token = [&](int tt) {
            const float4* B4 = reinterpret_cast<const float4*>(sB[buf][tt]);
            const float4* C4 = reinterpret_cast<const float4*>(sC[buf][tt]);
            const float a = sa[buf][tt];
            const float dt = sdt[buf][tt];
            float xv[CPT], u[CPT], part[CPT][4];
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                xv[c] = sx[buf][tt][col + c];
                u[c] = dt * xv[c];
                part[c][0] = part[c][1] = part[c][2] = part[c][3] = 0.f;
            }
#pragma unroll
            for (int k = 0; k < NC; ++k) {
                const float4 bv = B4[k * LANES + l], cv = C4[k * LANES + l];
#pragma unroll
                for (int c = 0; c < CPT; ++c) {
                    s[c][4 * k + 0] = fmaf(a, s[c][4 * k + 0], bv.x * u[c]);
                    s[c][4 * k + 1] = fmaf(a, s[c][4 * k + 1], bv.y * u[c]);
                    s[c][4 * k + 2] = fmaf(a, s[c][4 * k + 2], bv.z * u[c]);
                    s[c][4 * k + 3] = fmaf(a, s[c][4 * k + 3], bv.w * u[c]);
                    part[c][0] = fmaf(s[c][4 * k + 0], cv.x, part[c][0]);
                    part[c][1] = fmaf(s[c][4 * k + 1], cv.y, part[c][1]);
                    part[c][2] = fmaf(s[c][4 * k + 2], cv.z, part[c][2]);
                    part[c][3] = fmaf(s[c][4 * k + 3], cv.w, part[c][3]);
                }
            }
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                float sum = (part[c][0] + part[c][1]) + (part[c][2] + part[c][3]);
#pragma unroll
                for (int w = 1; w < LANES; w <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, w);
                if (l == 0 && j + c < P) yp[c] = fmaf(dh, xv[c], sum);
            }
            yp += ystep;
        };
        if (cnt == TT) {
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) token(tt);
        } else {
            for (int tt = 0; tt < cnt; ++tt) token(tt);
        }
        __syncthreads();                                   // this buffer is asked for again in the next round
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int c = 0; c < CPT; ++c)
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int n = ((i >> 2) * LANES + l) * 4 + (i & 3);
            if (n < N && j + c < P) Sh[(long long)n * P + j + c] = s[c][i];
        }
}

// One block a (token, part of the row): v = y silu(z); v / rms(v) * w * scale.  A thread keeps up to eight of
// its values between the two passes; a part wider than that is read twice.
template <typename TO>
__global__ void __launch_bounds__(128)
ssm_finish_kernel(const float* __restrict__ y, const float* __restrict__ p, SsmShape s, const float* __restrict__ w,
                  TO* __restrict__ out, int n_tokens, int n_groups, float eps, float scale) {
    __shared__ float red[33];
    pdl_trigger();
    pdl_wait();
    const long long t = blockIdx.x / n_groups;
    const int grp = blockIdx.x % n_groups;
    const int inner = s.H * s.P, per = inner / n_groups;
    const int c0 = grp * per;
    auto gated = [&](int c) -> float {
        const float z = ssm_proj(p, s, t, s.z_off + c);
        return y[t * inner + c] * z / (1.0f + expf(-z));
    };
    float keep[8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = threadIdx.x + i * blockDim.x;
        keep[i] = e < per ? gated(c0 + e) : 0.f;
        ss += keep[i] * keep[i];
    }
    for (int e = threadIdx.x + 8 * blockDim.x; e < per; e += blockDim.x) { const float v = gated(c0 + e); ss += v * v; }
    ss = block_sum(ss, red);
    const float inv = inv_rms(ss, (float)per, eps) * scale;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = threadIdx.x + i * blockDim.x;
        if (e < per) out[t * inner + c0 + e] = from_f32<TO>(keep[i] * inv * w[c0 + e]);
    }
    for (int e = threadIdx.x + 8 * blockDim.x; e < per; e += blockDim.x)
        out[t * inner + c0 + e] = from_f32<TO>(gated(c0 + e) * inv * w[c0 + e]);
}

// ---------------------------------------------------------------------------------------
// shape: [H, P, N, G, taps, z_off, x_off, b_off, c_off, dt_off] (10 ints)
static int read_shape(const int* shape, long long ldp, int n_parts, long long part_stride, SsmShape& s) {
    s.H = shape[0]; s.P = shape[1]; s.N = shape[2]; s.G = shape[3]; s.taps = shape[4];
    s.z_off = shape[5]; s.x_off = shape[6]; s.b_off = shape[7]; s.c_off = shape[8]; s.dt_off = shape[9];
    s.ldp = ldp; s.n_parts = n_parts; s.part_stride = part_stride;
    if (s.H <= 0 || s.G <= 0 || s.H % s.G || s.P <= 0 || s.N <= 0 || s.N > 256 || s.taps < 1 || s.taps > SSM_MAX_TAPS ||
        s.H > 65535 || n_parts < 1) return UB_ERR_ARG;
    // the convolution's channels are consecutive columns: x, then B, then C
    if (s.b_off != s.x_off + s.H * s.P || s.c_off != s.b_off + s.G * s.N) return UB_ERR_ARG;
    return 0;
}

UB_API int ub_ssm_prepare(const float* p, long long ldp, int n_parts, long long part_stride, const int* shape,
                          const float* conv_w, const float* conv_b, float* conv_state, int update_state, const float* dt_bias,
                          const float* a_log, const int* tok_seq, const int* seq_start, const int* seq_slot, float* xbc,
                          float* dtv, float* dec, int n_tokens, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    SsmShape s;
    if (int rc = read_shape(shape, ldp, n_parts, part_stride, s)) return rc;
    const long long n = (long long)n_tokens * (s.H * s.P + 2 * s.G * s.N + s.H);
    return (int)ub_launch_dependent(ssm_prepare_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, p, s, conv_w, conv_b,
                                    conv_state, update_state, dt_bias, a_log, tok_seq, seq_start, seq_slot, xbc, dtv, dec, n_tokens);
}

UB_API int ub_ssm_conv_state_update(const float* p, long long ldp, int n_parts, long long part_stride, const int* shape,
                                    float* conv_state, const int* seq_start, const int* seq_slot, int n_seqs, cudaStream_t st) {
    if (n_seqs <= 0) return 0;
    SsmShape s;
    if (int rc = read_shape(shape, ldp, n_parts, part_stride, s)) return rc;
    if (s.taps <= 1) return 0;
    const long long n = (long long)n_seqs * (s.H * s.P + 2 * s.G * s.N);
    return (int)ub_launch_dependent(ssm_conv_state_update_kernel, dim3((unsigned)((n + 127) / 128)), dim3(128), 0, st, p, s,
                                    conv_state, seq_start, seq_slot, n_seqs);
}

UB_API int ub_ssm_scan(const float* xbc, const float* dtv, const float* dec, const float* Dw, float* y, float* S,
                       const int* seq_start, const int* seq_slot, int n_seqs, int n_tokens, int H, int P, int N, int G,
                       int sm_count, cudaStream_t st) {
    if (n_seqs <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || P <= 0 || N <= 0 || N > 256 || H > 65535 || n_seqs > 65535) return UB_ERR_ARG;
    const int lanes = N >= 128 ? 32 : (N >= 64 ? 16 : 8);
    // two columns a thread where that still leaves about one and a half blocks for every multiprocessor (measured at
    // 2,048 tokens, state 128, heads of 64: 64 heads 875 -> 681 us with two, 32 heads 568 -> 591 us)
    const long long blocks2 = (long long)((P + 256 / lanes * 2 - 1) / (256 / lanes * 2)) * H * n_seqs;
    const int cpt = blocks2 * 2 >= 3LL * (sm_count > 0 ? sm_count : 148) ? 2 : 1;
    const int cols = 256 / lanes * cpt;
    const dim3 grid((P + cols - 1) / cols, H, n_seqs), block(256);
    const int per = (N + lanes - 1) / lanes;               // at most 8: N <= 256
    const bool vec = N % 4 == 0 && P % 4 == 0 && (((uintptr_t)xbc) & 15) == 0;
    cudaError_t e;
    // a step of more than one token a sequence: an ordinary launch, so that the blocks, each busy for the whole step, are
    // spread over idle SMs instead of being placed where the kernel before happens to drain first (as the delta rule's scan)
    const bool dep = n_tokens <= n_seqs;
#define GO4(RR, LL, CC, VV) do { \
        constexpr size_t smem = SsmScanLayout<RR, LL, CC>::BYTES; \
        static bool attr_done = false; \
        if (!attr_done) { \
            e = cudaFuncSetAttribute(ssm_scan_kernel<RR, LL, CC, VV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e; \
            attr_done = true; \
        } \
        e = ub_launch_ordered(dep, ssm_scan_kernel<RR, LL, CC, VV>, grid, block, smem, st, xbc, dtv, dec, Dw, y, S, seq_start, seq_slot, H, P, N, G); \
    } while (0)
#define GO3(RR, LL, CC) do { if (vec) GO4(RR, LL, CC, true); else GO4(RR, LL, CC, false); } while (0)
#define GO2(RR, LL) do { if (cpt == 2) GO3(RR, LL, 2); else GO3(RR, LL, 1); } while (0)
#define GO(RR) do { if (lanes == 32) GO2(RR, 32); else if (lanes == 16) GO2(RR, 16); else GO2(RR, 8); } while (0)
    if (per <= 4) GO(4); else GO(8);
#undef GO
#undef GO2
#undef GO3
#undef GO4
    return (int)e;
}

UB_API int ub_ssm_finish(const float* y, const float* p, long long ldp, int n_parts, long long part_stride, const int* shape,
                         const float* w, void* out, int out_dtype, int n_tokens, int n_groups, float eps, float scale,
                         cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    SsmShape s;
    if (int rc = read_shape(shape, ldp, n_parts, part_stride, s)) return rc;
    if (n_groups < 1 || (s.H * s.P) % n_groups) return UB_ERR_ARG;
    const long long blocks = (long long)n_tokens * n_groups;
    if (blocks > 0x7fffffffLL) return UB_ERR_ARG;
    const unsigned grid = (unsigned)blocks;
    cudaError_t e;
    if (out_dtype == UB_F32)
        e = ub_launch_dependent(ssm_finish_kernel<float>, dim3(grid), dim3(128), 0, st, y, p, s, w, (float*)out, n_tokens, n_groups, eps, scale);
    else if (out_dtype == UB_BF16)
        e = ub_launch_dependent(ssm_finish_kernel<__nv_bfloat16>, dim3(grid), dim3(128), 0, st, y, p, s, w, (__nv_bfloat16*)out, n_tokens, n_groups, eps, scale);
    else return UB_ERR_UNSUPPORTED;
    return (int)e;
}

// ---------------------------------------------------------------------------------------
// The selective scan with a decay for every (channel, state element) (the first Mamba form).  For channel c with the step
// size dt = softplus(dtp + dt_bias[c]), the input x (convolved, activated), and the token's B and C rows of N numbers:
//     S[c, n] <- exp(dt A[c, n]) S[c, n] + dt x B[n];    y = sum_n S[c, n] C[n] + D[c] x;    out = y * silu(z)
// A = -exp(A_log) is made once at load.  A block of 128 threads takes 128 / LANES channels of one sequence; LANES lanes
// hold one channel's N state elements (NR = ceil(N / LANES) each, element n with lane n % LANES) in registers for the step.  Tokens
// come through shared memory a stage at a time: while one stage is worked on, the next one's B and C rows and the
// channels' dt, x and z are on their way from global memory into registers (softplus and the gate's SiLU are taken
// there, off the chain from token to token), and a stage's results leave in whole rows.  Everything is float32; x comes
// in the activation type (it is a convolution's output), z as float32 sums of the input product's K slices.
// ---------------------------------------------------------------------------------------
// 2^x by the hardware's approximation (about 2^-22 relative): the decay of a state element, taken sixteen times a token and lane
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <typename TX, int LANES, int NR>
__global__ void __launch_bounds__(128)
mamba1_scan_kernel(const TX* __restrict__ x, const float* __restrict__ dtp, const float* __restrict__ dt_bias,
                   const float* __restrict__ bc, long long ldbc, int b_off, int c_off, const float* __restrict__ A,
                   const float* __restrict__ Dskip, const float* __restrict__ z, long long ldz, int z_parts, long long z_part_stride,
                   TX* __restrict__ out, float* __restrict__ S, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                   int inner, int N) {
    constexpr int CH = 128 / LANES;                        // channels a block
    constexpr int NS = LANES * NR;                         // state elements, padded
    constexpr int TT = NS <= 32 ? 16 : 8;                  // tokens a stage
    constexpr int ROW = 2 * NS + 3 * CH;                   // a token in shared memory: B, C, then dt, x and the gate of the channels
    constexpr int PER = (TT * ROW + 127) / 128;
    constexpr int U = NR <= 4 ? 4 : 2;                     // tokens whose decays are formed together
    __shared__ float sm[2][TT][ROW];
    __shared__ float sp[TT][CH * (LANES + 1)];             // a lane's share of a token's read-out (a channel's lanes one bank on)
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, cl = tid / LANES, q = tid % LANES;
    const int b = blockIdx.y, c0 = blockIdx.x * CH, c = c0 + cl;
    const int t0 = seq_start[b], t1 = seq_start[b + 1];
    if (t0 >= t1) return;
    float* Sc = S + ((long long)seq_slot[b] * inner + c) * N;
    float s[NR], a[NR];
#pragma unroll
    for (int i = 0; i < NR; ++i) {
        const int n = i * LANES + q;
        const bool in = c < inner && n < N;
        s[i] = in ? Sc[n] : 0.f;
        a[i] = in ? A[(long long)c * N + n] * 1.4426950408889634f : 0.f;      // powers of two
    }
    // What this thread brings into a stage is the same from stage to stage but for the first token: the places are worked
    // out once (a pointer at token 0, a stride a token, what is done to the number), so that a stage's fetch is loads only.
    float reg[PER];
    const float* src[PER];                                 // float sources: B, C, the step size's sums, the gate's sums
    const TX* srcx[PER];                                   // x comes in the activation type
    long long step[PER];
    float add[PER];
    int kind[PER];                                         // 0 nothing to bring, 1 a float as it is, 2 step size (softplus), 3 x, 4 gate (SiLU)
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = tid + i * 128;
        const int tt = e / ROW, j = e % ROW;
        src[i] = nullptr; srcx[i] = nullptr; step[i] = 0; add[i] = 0.f; kind[i] = 0;
        if (tt >= TT) continue;
        if (j < 2 * NS) {
            const int n = j < NS ? j : j - NS;
            if (n < N) { kind[i] = 1; step[i] = ldbc; src[i] = bc + tt * ldbc + (j < NS ? b_off : c_off) + n; }
        } else {
            const int k = j - 2 * NS, cc = c0 + k % CH;
            if (cc < inner) {
                if (k < CH) { kind[i] = 2; step[i] = inner; src[i] = dtp + (long long)tt * inner + cc; add[i] = dt_bias[cc]; }
                else if (k < 2 * CH) { kind[i] = 3; step[i] = inner; srcx[i] = x + (long long)tt * inner + cc; }
                else { kind[i] = 4; step[i] = ldz; src[i] = z + (long long)tt * ldz + cc; }
            }
        }
    }
    auto fetch = [&](int base) {                           // a stage's numbers on their way into registers: loads only
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int tt = (tid + i * 128) / ROW;
            float v = 0.f;
            if (kind[i] && base + tt < t1) {
                if (kind[i] == 3) v = to_f32<TX>(srcx[i][(long long)base * step[i]]);
                else {
                    // (a load the compiler may not move down to where the number is used, behind the stage's arithmetic)
                    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(src[i] + (long long)base * step[i]));
                    if (kind[i] == 4) for (int p = 1; p < z_parts; ++p) v += src[i][(long long)base * step[i] + p * z_part_stride];
                }
            }
            reg[i] = v;
        }
    };
    auto stash = [&](int buf, int base) {                  // ... and into shared memory, the step size through softplus, the gate through SiLU
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int e = tid + i * 128;
            if (e >= TT * ROW) continue;
            float v = reg[i];
            if (base + e / ROW >= t1) v = 0.f;             // past the sequence's end: a step size of zero leaves the state as it is
            else if (kind[i] == 2) { v += add[i]; v = v > 20.f ? v : log1pf(expf(v)); }
            else if (kind[i] == 4) v = v / (1.0f + expf(-v));
            (&sm[buf][0][0])[e] = v;
        }
    };
    fetch(t0);
    stash(0, t0);
    __syncthreads();
    int buf = 0;
    for (int base = t0; base < t1; base += TT, buf ^= 1) {
        const int n_tok = min(TT, t1 - base);
        const bool more = base + TT < t1;
        if (more) fetch(base + TT);
        // Tokens past the sequence's end are zeros in shared memory (decay 1, nothing written), so a stage is always walked
        // whole.  Four tokens at a time: their decays and inputs first (independent of one another), then the chain from
        // token to token, which is one multiply-add a state element; a lane's share of the read-out goes to shared memory
        // and is summed over the lanes behind the stage.
#pragma unroll
        for (int t4 = 0; t4 < TT; t4 += U) {
            float dA[U][NR], in[U][NR];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const float* row = sm[buf][t4 + u];
                const float dt = row[2 * NS + cl];
                const float dx = dt * row[2 * NS + CH + cl];
#pragma unroll
                for (int i = 0; i < NR; ++i) {
                    dA[u][i] = fast_exp2(dt * a[i]);
                    in[u][i] = dx * row[i * LANES + q];
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const float* row = sm[buf][t4 + u];
                float y = 0.f;
#pragma unroll
                for (int i = 0; i < NR; ++i) {
                    s[i] = fmaf(dA[u][i], s[i], in[u][i]);
                    y = fmaf(s[i], row[NS + i * LANES + q], y);
                }
                sp[t4 + u][cl * (LANES + 1) + q] = y;      // [token][channel of the block][lane]
            }
        }
        if (more) stash(buf ^ 1, base + TT);               // (that buffer's readers passed the barrier at the end of the last round)
        __syncthreads();
        for (int e = tid; e < n_tok * CH; e += 128) {
            const int tt = e / CH, k = e % CH;
            if (c0 + k >= inner) continue;
            float y = 0.f;
#pragma unroll
            for (int l = 0; l < LANES; ++l) y += sp[tt][k * (LANES + 1) + l];
            const float* row = sm[buf][tt];
            y = fmaf(Dskip[c0 + k], row[2 * NS + CH + k], y) * row[2 * NS + 2 * CH + k];
            out[(long long)(base + tt) * inner + c0 + k] = from_f32<TX>(y);
        }
        __syncthreads();
    }
    if (c < inner) {
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int n = i * LANES + q;
            if (n < N) Sc[n] = s[i];
        }
    }
}

// ---------------------------------------------------------------------------------------
// The same scan for steps of many tokens a sequence, as three kernels: what is a function of one (token, channel) alone
// is taken out of the chain from token to token.
//   mamba1_pre     dt = softplus(dtp + dt_bias) (in place) and dx = dt * x, float32
//   mamba1_chain   the recurrence over copies (cp.async, two stages in flight) of dt, dx, B and C: per token and state
//                  element one exponential and three multiply-adds; the sum over the state goes out in float32
//   mamba1_post    out = (sum + D x) * silu(z)
// The arithmetic and its order are those of the one-kernel form above.
// ---------------------------------------------------------------------------------------
template <typename TX>
__global__ void mamba1_pre_kernel(float* __restrict__ dtp, const float* __restrict__ dt_bias, const TX* __restrict__ x,
                                  float* __restrict__ dx, long long n, int inner) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float pre = dtp[i] + dt_bias[i % inner];
    const float dt = pre > 20.f ? pre : log1pf(expf(pre));
    dtp[i] = dt;
    dx[i] = dt * to_f32<TX>(x[i]);
}

__device__ __forceinline__ void m1_cp4(float* dst, const float* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}

template <int LANES, int NR>
__global__ void __launch_bounds__(128)
mamba1_chain_kernel(const float* __restrict__ dt, const float* __restrict__ dx, const float* __restrict__ bc, long long ldbc,
                    int b_off, int c_off, const float* __restrict__ A, float* __restrict__ ysum, float* __restrict__ S,
                    const int* __restrict__ seq_start, const int* __restrict__ seq_slot, int inner, int N) {
    constexpr int CH = 128 / LANES;
    constexpr int NS = LANES * NR;
    constexpr int TT = NS <= 32 ? 16 : 8;
    constexpr int ROW = 2 * NS + 2 * CH;                   // a token in shared memory: B, C, then dt and dx of the channels
    constexpr int U = NR <= 4 ? 4 : 2;
    __shared__ float sm[2][TT][ROW];
    __shared__ float sp[TT][CH * (LANES + 1)];
    const int tid = threadIdx.x, cl = tid / LANES, q = tid % LANES;
    const int b = blockIdx.y, c0 = blockIdx.x * CH, c = c0 + cl;
    const int t0 = seq_start[b], t1 = seq_start[b + 1];
    if (t0 >= t1) return;
    float* Sc = S + ((long long)seq_slot[b] * inner + c) * N;
    float s[NR], a[NR];
#pragma unroll
    for (int i = 0; i < NR; ++i) {
        const int n = i * LANES + q;
        const bool in = c < inner && n < N;
        s[i] = in ? Sc[n] : 0.f;
        a[i] = in ? A[(long long)c * N + n] * 1.4426950408889634f : 0.f;
    }
    auto fetch = [&](int base, int buf) {                  // copies for the tokens there are, zeros behind the sequence's end and past the sizes
        for (int e = tid; e < TT * ROW; e += 128) {
            const int tt = e / ROW, j = e % ROW;
            const long long t = (long long)base + tt;
            float* dst = &sm[buf][tt][j];
            const float* src = nullptr;
            if (t < t1) {
                if (j < 2 * NS) {
                    const int n = j < NS ? j : j - NS;
                    if (n < N) src = bc + t * ldbc + (j < NS ? b_off : c_off) + n;
                } else {
                    const int k = j - 2 * NS, cc = c0 + k % CH;
                    if (cc < inner) src = (k < CH ? dt : dx) + t * inner + cc;
                }
            }
            if (src) m1_cp4(dst, src); else *dst = 0.f;
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch(t0, 0);
    int buf = 0;
    for (int base = t0; base < t1; base += TT, buf ^= 1) {
        const int n_tok = min(TT, t1 - base);
        if (base + TT < t1) {
            fetch(base + TT, buf ^ 1);                     // (that buffer's readers passed the barrier at the end of the last round)
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
#pragma unroll
        for (int t4 = 0; t4 < TT; t4 += U) {
            float dA[U][NR], in[U][NR];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const float* row = sm[buf][t4 + u];
                const float dtv = row[2 * NS + cl], dxv = row[2 * NS + CH + cl];
#pragma unroll
                for (int i = 0; i < NR; ++i) {
                    dA[u][i] = fast_exp2(dtv * a[i]);
                    in[u][i] = dxv * row[i * LANES + q];
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const float* row = sm[buf][t4 + u];
                float y = 0.f;
#pragma unroll
                for (int i = 0; i < NR; ++i) {
                    s[i] = fmaf(dA[u][i], s[i], in[u][i]);
                    y = fmaf(s[i], row[NS + i * LANES + q], y);
                }
                sp[t4 + u][cl * (LANES + 1) + q] = y;
            }
        }
        __syncthreads();
        for (int e = tid; e < n_tok * CH; e += 128) {
            const int tt = e / CH, k = e % CH;
            if (c0 + k >= inner) continue;
            float y = 0.f;
#pragma unroll
            for (int l = 0; l < LANES; ++l) y += sp[tt][k * (LANES + 1) + l];
            ysum[(long long)(base + tt) * inner + c0 + k] = y;
        }
        __syncthreads();
    }
    if (c < inner) {
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int n = i * LANES + q;
            if (n < N) Sc[n] = s[i];
        }
    }
}

template <typename TX>
__global__ void mamba1_post_kernel(const float* __restrict__ ysum, const TX* __restrict__ x, const float* __restrict__ Dskip,
                                   const float* __restrict__ z, long long ldz, int z_parts, long long z_part_stride,
                                   TX* __restrict__ out, long long n, int inner) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long t = i / inner;
    const int c = (int)(i % inner);
    float zv = 0.f;
    for (int p = 0; p < z_parts; ++p) zv += z[p * z_part_stride + t * ldz + c];
    const float y = fmaf(Dskip[c], to_f32<TX>(x[i]), ysum[i]);
    out[i] = from_f32<TX>(y * (zv / (1.0f + expf(-zv))));
}

// work: two float32 arrays [n_tokens, inner] (dx and the sums); dtp is overwritten with the step sizes
UB_API int ub_mamba1_scan_staged(const void* x, int x_dtype, float* dtp, const float* dt_bias, const float* bc, long long ldbc,
                                 int b_off, int c_off, const float* A, const float* Dskip, const float* z, long long ldz,
                                 int z_parts, long long z_part_stride, void* out, int out_dtype, float* S, const int* seq_start,
                                 const int* seq_slot, int n_seqs, int n_tokens, int inner, int N, float* work, cudaStream_t st) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (inner <= 0 || N <= 0 || N > 256 || n_seqs > 65535 || z_parts < 1 || x_dtype != out_dtype || !work) return UB_ERR_ARG;
    const long long n = (long long)n_tokens * inner;
    float* dx = work;
    float* ysum = work + n;
    const dim3 egrid((unsigned)((n + 255) / 256)), eblock(256);
    cudaError_t e;
    if (x_dtype == UB_F32) e = ub_launch_dependent(mamba1_pre_kernel<float>, egrid, eblock, 0, st, dtp, dt_bias, (const float*)x, dx, n, inner);
    else if (x_dtype == UB_BF16) e = ub_launch_dependent(mamba1_pre_kernel<__nv_bfloat16>, egrid, eblock, 0, st, dtp, dt_bias, (const __nv_bfloat16*)x, dx, n, inner);
    else return UB_ERR_UNSUPPORTED;
    if (e != cudaSuccess) return (int)e;
    const int lanes = N <= 4 ? 4 : 16;
    const int ch = 128 / lanes;
    const dim3 grid((unsigned)((inner + ch - 1) / ch), n_seqs), block(128);
    const int nr = (N + lanes - 1) / lanes;
    // an ordinary launch, behind the end of the kernels before it: its blocks are busy for the whole step, as the other scans'
#define GO(LL, NRR) e = ub_launch_ordered(false, mamba1_chain_kernel<LL, NRR>, grid, block, 0, st, (const float*)dtp, (const float*)dx, bc, ldbc, \
                                          b_off, c_off, A, ysum, S, seq_start, seq_slot, inner, N)
    if (lanes == 4) GO(4, 1);
    else if (nr <= 1) GO(16, 1); else if (nr <= 2) GO(16, 2); else if (nr <= 4) GO(16, 4); else if (nr <= 8) GO(16, 8); else GO(16, 16);
#undef GO
    if (e != cudaSuccess) return (int)e;
    if (x_dtype == UB_F32) e = ub_launch_ordered(false, mamba1_post_kernel<float>, egrid, eblock, 0, st, (const float*)ysum, (const float*)x, Dskip, z, ldz, z_parts, z_part_stride, (float*)out, n, inner);
    else e = ub_launch_ordered(false, mamba1_post_kernel<__nv_bfloat16>, egrid, eblock, 0, st, (const float*)ysum, (const __nv_bfloat16*)x, Dskip, z, ldz, z_parts, z_part_stride, (__nv_bfloat16*)out, n, inner);
    return (int)e;
}

// One token a sequence: four lanes a (sequence, channel), a lane the state elements n = q, q + 4, ...; nothing is staged.
template <typename TX>
__global__ void __launch_bounds__(128)
mamba1_step_kernel(const TX* __restrict__ x, const float* __restrict__ dtp, const float* __restrict__ dt_bias,
                   const float* __restrict__ bc, long long ldbc, int b_off, int c_off, const float* __restrict__ A,
                   const float* __restrict__ Dskip, const float* __restrict__ z, long long ldz, int z_parts, long long z_part_stride,
                   TX* __restrict__ out, float* __restrict__ S, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                   int inner, int N) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.y, q = threadIdx.x & 3;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) >> 2;
    const bool live = c < inner;                           // (every lane stays for the exchanges)
    const long long t = seq_start[b];
    const int cc = live ? c : 0;
    const float pre = dtp[t * inner + cc] + dt_bias[cc];
    const float dt = pre > 20.f ? pre : log1pf(expf(pre));
    const float xv = to_f32<TX>(x[t * inner + cc]);
    const float dx = dt * xv;
    float* Sc = S + ((long long)seq_slot[b] * inner + cc) * N;
    const float* Ac = A + (long long)cc * N;
    const float* Bt = bc + t * ldbc + b_off;
    const float* Ct = bc + t * ldbc + c_off;
    float y = 0.f;
    if (live) {
        for (int n = q; n < N; n += 4) {
            const float sn = fmaf(fast_exp2(dt * Ac[n] * 1.4426950408889634f), Sc[n], dx * Bt[n]);
            Sc[n] = sn;
            y = fmaf(sn, Ct[n], y);
        }
    }
    y += __shfl_xor_sync(0xffffffffu, y, 1);
    y += __shfl_xor_sync(0xffffffffu, y, 2);
    if (live && q == 0) {
        float zv = 0.f;
        for (int p = 0; p < z_parts; ++p) zv += z[p * z_part_stride + t * ldz + c];
        out[t * inner + c] = from_f32<TX>(fmaf(Dskip[c], xv, y) * (zv / (1.0f + expf(-zv))));
    }
}

UB_API int ub_mamba1_scan(const void* x, int x_dtype, const float* dtp, const float* dt_bias, const float* bc, long long ldbc,
                          int b_off, int c_off, const float* A, const float* Dskip, const float* z, long long ldz, int z_parts,
                          long long z_part_stride, void* out, int out_dtype, float* S, const int* seq_start, const int* seq_slot,
                          int n_seqs, int n_tokens, int inner, int N, cudaStream_t st) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (inner <= 0 || N <= 0 || N > 256 || n_seqs > 65535 || z_parts < 1 || x_dtype != out_dtype) return UB_ERR_ARG;
    if (n_tokens == n_seqs) {                               // one token a sequence (every sequence of a step brings at least one)
        const dim3 sgrid((unsigned)((inner * 4 + 127) / 128), n_seqs), sblock(128);
        cudaError_t e;
        if (x_dtype == UB_F32) e = ub_launch_dependent(mamba1_step_kernel<float>, sgrid, sblock, 0, st, (const float*)x, dtp, dt_bias, bc, ldbc, b_off, c_off, A, Dskip, z, ldz, z_parts, z_part_stride, (float*)out, S, seq_start, seq_slot, inner, N);
        else if (x_dtype == UB_BF16) e = ub_launch_dependent(mamba1_step_kernel<__nv_bfloat16>, sgrid, sblock, 0, st, (const __nv_bfloat16*)x, dtp, dt_bias, bc, ldbc, b_off, c_off, A, Dskip, z, ldz, z_parts, z_part_stride, (__nv_bfloat16*)out, S, seq_start, seq_slot, inner, N);
        else return UB_ERR_UNSUPPORTED;
        return (int)e;
    }
    // lanes a channel: four for the smallest states, else sixteen (more warps with shorter chains: the kernel is bound by
    // the chain from token to token, not by bytes)
    const int lanes = N <= 4 ? 4 : 16;
    const int ch = 128 / lanes;
    const dim3 grid((unsigned)((inner + ch - 1) / ch), n_seqs), block(128);
    const int nr = (N + lanes - 1) / lanes;
    // a step of more than one token a sequence starts behind the end of the kernels before it, as the other scans do
    const bool dep = n_tokens <= n_seqs;
    cudaError_t e = cudaErrorInvalidValue;
#define GO3(TX, LL, NRR) e = ub_launch_ordered(dep, mamba1_scan_kernel<TX, LL, NRR>, grid, block, 0, st, (const TX*)x, dtp, dt_bias, bc, ldbc, b_off, \
                                               c_off, A, Dskip, z, ldz, z_parts, z_part_stride, (TX*)out, S, seq_start, seq_slot, inner, N)
#define GO(LL, NRR) do { if (x_dtype == UB_F32) GO3(float, LL, NRR); else if (x_dtype == UB_BF16) GO3(__nv_bfloat16, LL, NRR); else return UB_ERR_UNSUPPORTED; } while (0)
    if (lanes == 4) GO(4, 1);
    else if (nr <= 1) GO(16, 1); else if (nr <= 2) GO(16, 2); else if (nr <= 4) GO(16, 4); else if (nr <= 8) GO(16, 8); else GO(16, 16);
#undef GO
#undef GO3
    return (int)e;
}
