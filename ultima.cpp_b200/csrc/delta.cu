// The gated delta-rule mixer: a recurrent layer whose state is, for every head, a matrix S [D, E]
// (D key channels, E value channels) in float32, plus the last inputs of a short causal convolution.
//
// For one token of one head, with unit vectors q (scaled) and k, a value v, a write strength b in
// (0, 1) and a decay a[d] in (0, 1) for every key channel:
//     S[d, :] *= a[d];   u = b * (v - S^T k);   S += k u^T;   o = S^T q
// so the read-out sees the token's own write.  Every column of S evolves on its own, which is what
// the scan kernel uses: a group of eight lanes holds one column, tokens are taken in order.
//
// Four kernels, for prompts and single tokens alike (a step's tokens of one sequence are rows
// seq_start[s] .. seq_start[s + 1] of the packed batch; state rows are slot numbers):
//   delta_prepare      short convolution + SiLU of q, k, v; unit vectors; write strength; decay
//   conv_state_update  the convolution's last inputs, carried to the next step
//   delta_scan         the recurrence
//   delta_finish       per-head RMS norm of o, weight, output gate (sigmoid or SiLU of the gate's sums)
// The decay is one number a head and key channel (its sums come in a matrix of their own, ``dpre``), or one
// number a head whose sums are a column range of the projection row (``a_off`` >= 0; the bias then has one
// entry a head).
// Everything is float32; the projections come in as float32 sums of the products (for few tokens as the
// partial sums of K slices, which the kernels add up as they read).
#include "common.cuh"
#include <stdlib.h>

constexpr int MAX_TAPS = 16;

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }

struct DeltaShape {
    int H, G, D, E;          // heads, q/k heads, key size, value size
    int taps;                // convolution length (the last tap is the current token's)
    int q_off, k_off, v_off, b_off;   // columns of a projection row
    int a_off;               // >= 0: one decay a head, its sums in the H columns from here on; < 0: one a key channel, from dpre
    long long ldp;           // row stride of the projections
    int n_parts;             // the projection row is the sum of this many partial results ...
    long long part_stride;   // ... this many elements apart
};

__device__ __forceinline__ float proj_at(const float* __restrict__ p, const DeltaShape& s, long long t, int c) {
    float v = 0.f;
    for (int i = 0; i < s.n_parts; ++i) v += p[i * s.part_stride + t * s.ldp + c];
    return v;
}

// One warp a (token, unit); units of a token: G query heads, G key heads, H value heads (which also
// make the head's write strength and decay).  ``update_state`` (only when every sequence brings ONE token, so
// that a channel's state has this lane as its only reader): the convolution's state moves on here, and
// conv_state_update is not launched.
__global__ void __launch_bounds__(128)
delta_prepare_kernel(const float* __restrict__ p, DeltaShape s, const float* __restrict__ conv_w,
                     float* conv_state, int update_state, const float* __restrict__ dpre,
                     const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                     const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
                     const int* __restrict__ seq_slot, float* __restrict__ qn, float* __restrict__ kn,
                     float* __restrict__ vc, float* __restrict__ beta, float* __restrict__ dec,
                     int n_tokens, float unit_eps, float q_scale) {
    pdl_trigger();
    pdl_wait();
    const int units = 2 * s.G + s.H;
    const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)n_tokens * units) return;
    const int t = (int)(wid / units), unit = (int)(wid % units);
    const int seq = tok_seq[t];
    const int r = t - seq_start[seq];
    const int K = s.taps - 1;
    const int C = 2 * s.G * s.D + s.H * s.E;
    float* st = conv_state + (long long)seq_slot[seq] * K * C;

    auto conv_silu = [&](int c) -> float {
        float acc = 0.f;
        for (int j = K; j >= 0; --j) {                 // oldest input first
            const float w = conv_w[(long long)c * s.taps + (s.taps - 1 - j)];
            const float x = (r - j >= 0) ? proj_at(p, s, t - j, c) : st[(long long)(K + r - j) * C + c];
            acc = fmaf(w, x, acc);
            if (update_state && j < K) st[(long long)(K - 1 - j) * C + c] = x;     // r = 0: the input j back becomes j + 1 back
        }
        return acc * sigmoidf_(acc);
    };

    if (unit < 2 * s.G) {
        const bool is_q = unit < s.G;
        const int head = is_q ? unit : unit - s.G;
        const int c0 = (is_q ? s.q_off : s.k_off) + head * s.D;      // q_off = 0 and k_off = G * D: columns are channels
        float vals[8];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int d = lane + 32 * i;
            vals[i] = d < s.D ? conv_silu(c0 + d) : 0.f;
            ss += vals[i] * vals[i];
        }
        ss = warp_sum(ss);
        const float inv = (is_q ? q_scale : 1.0f) / sqrtf(ss + unit_eps);
        float* o = (is_q ? qn : kn) + (long long)t * s.G * s.D + head * s.D;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int d = lane + 32 * i;
            if (d < s.D) o[d] = vals[i] * inv;
        }
        return;
    }
    const int h = unit - 2 * s.G;
    for (int e = lane; e < s.E; e += 32)
        vc[(long long)t * s.H * s.E + h * s.E + e] = conv_silu(s.v_off + h * s.E + e);
    if (lane == 0) beta[(long long)t * s.H + h] = sigmoidf_(proj_at(p, s, t, s.b_off + h));
    const float rate = expf(a_log[h]);
    if (s.a_off >= 0) {
        const float a = expf(-rate * softplusf_(proj_at(p, s, t, s.a_off + h) + dt_bias[h]));
        for (int d = lane; d < s.D; d += 32) dec[(long long)t * s.H * s.D + h * s.D + d] = a;
        return;
    }
    for (int d = lane; d < s.D; d += 32) {
        const long long c = (long long)t * s.H * s.D + h * s.D + d;
        dec[c] = expf(-rate * softplusf_(dpre[c] + dt_bias[h * s.D + d]));
    }
}

// One thread a (sequence, channel): the last taps - 1 inputs of what the state held followed by the step's.
__global__ void conv_state_update_kernel(const float* __restrict__ p, DeltaShape s, float* __restrict__ conv_state,
                                         const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                                         int n_seqs, int C, int taps) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_seqs * C) return;
    const int b = (int)(i / C), c = (int)(i % C);
    const int K = taps - 1;
    const int first = seq_start[b], n = seq_start[b + 1] - first;
    float* st = conv_state + (long long)seq_slot[b] * K * C;
    float tmp[MAX_TAPS];
    for (int k = 0; k < K; ++k) {
        const int rel = n - K + k;
        tmp[k] = rel >= 0 ? proj_at(p, s, first + rel, c) : st[(long long)(K + rel) * C + c];
    }
    for (int k = 0; k < K; ++k) st[(long long)k * C + c] = tmp[k];
}

// The recurrence.  A block of 128 threads takes 128 / LANES value channels of one head of one sequence;
// LANES (8, 16 or 32) lanes hold one column of S, lane p the key channels of the float4 chunks p,
// p + LANES, ...: the lanes of a column read consecutive bytes of shared memory in one instruction, and a
// dot product over the key channels ends in log2(LANES) exchanges.  Tokens come through shared memory a
// few at a time, the next few asked for (cp.async) while these are worked on.
//
// The kernel is bound by latency, not by bytes or arithmetic: a token's update depends on the one before
// it through a chain of multiply, dot product, exchanges and update, and a warp issues in order.  The
// read-out o = S^T q is off that chain: its partial sums go to shared memory and are added up once for
// the tokens of a stage, and the loop over a full stage's tokens is unrolled.

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

// VEC: sizes are multiples of 4 and every array starts on a 16-byte boundary, so tokens are fetched in
// 16-byte copies, each thread keeping the same one or two places of a token's row for the whole launch.
//
// GEN: the generalised rule, in which a token removes along its unit key u at a rate of its own for every key channel and
// writes its raw key: with c = S_old^T u,  S[d, :] = w[d] S_old[d, :] - rem[d] c + kraw[d] v,  o = S^T q.  ``kn`` then holds
// u, ``dec`` holds w, ``rem`` = rate * u and ``kraw`` come as two more arrays of the keys' shape, and ``beta`` is not read.
template <int R, int SCAN_LANES, bool VEC, bool GEN>
__global__ void __launch_bounds__(128)
delta_scan_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ vc,
                  const float* __restrict__ beta, const float* __restrict__ dec, float* __restrict__ out,
                  float* __restrict__ S, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                  int H, int G, int D, int E, const float* __restrict__ rem, const float* __restrict__ kraw) {
    static_assert(R % 4 == 0, "a lane holds whole float4 chunks");
    constexpr int SCAN_COLS = 128 / SCAN_LANES;
    constexpr int DP = SCAN_LANES * R;
    constexpr int NC = R / 4;                             // chunks a lane
    constexpr int TT = DP <= 128 ? 8 : 4;                 // tokens a stage
    __shared__ __align__(16) float sq[2][TT][DP], sk[2][TT][DP], sa[2][TT][DP];
    __shared__ __align__(16) float sr[GEN ? 2 : 1][GEN ? TT : 1][GEN ? DP : 4], sw[GEN ? 2 : 1][GEN ? TT : 1][GEN ? DP : 4];
    __shared__ __align__(16) float sv[2][TT][SCAN_COLS];
    __shared__ float sb[2][TT];
    __shared__ float so[TT][128];                          // the read-out's partial sums, [token][lane of the column][column]
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x;
    const int col = tid / SCAN_LANES, p = tid % SCAN_LANES;
    const int h = blockIdx.y, b = blockIdx.z;
    const int g = h / (H / G);
    const int j = blockIdx.x * SCAN_COLS + col;
    const int t0 = seq_start[b], t1 = seq_start[b + 1];
    if (t0 >= t1) return;
    float* Sh = S + ((long long)seq_slot[b] * H + h) * D * E;
    float s[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int d = ((i >> 2) * SCAN_LANES + p) * 4 + (i & 3);
        s[i] = (d < D && j < E) ? Sh[(long long)d * E + j] : 0.f;
    }
    // columns past the sizes are constants that no copy ever touches
    for (int idx = tid; idx < 2 * TT * DP; idx += blockDim.x) {
        const int d = idx % DP;
        if (d >= D) {
            (&sq[0][0][0])[idx] = 0.f; (&sk[0][0][0])[idx] = 0.f; (&sa[0][0][0])[idx] = 1.f;
            if (GEN) { (&sr[0][0][0])[idx] = 0.f; (&sw[0][0][0])[idx] = 0.f; }
        }
    }
    for (int idx = tid; idx < 2 * TT * SCAN_COLS; idx += blockDim.x)
        if (blockIdx.x * SCAN_COLS + idx % SCAN_COLS >= E) (&sv[0][0][0])[idx] = 0.f;

    // this thread's places in a token's [q | k | decay] row of 3 * D / 4 chunks (VEC)
    constexpr int NARR = GEN ? 5 : 3, NSL = GEN ? 3 : 2;          // arrays of the keys' shape; places a thread may hold
    int my_arr[NSL], my_d[NSL];
    for (int sl = 0; sl < NSL; ++sl) { my_arr[sl] = -1; my_d[sl] = 0; }
    if (VEC) {
        const int d4 = D >> 2;
        for (int sl = 0; sl < NSL; ++sl) {
            const int c = tid + sl * (int)blockDim.x;
            if (c < NARR * d4) { my_arr[sl] = c / d4; my_d[sl] = (c % d4) * 4; }
        }
    }
    const float* qrow = qn + (long long)g * D;
    const float* krow = kn + (long long)g * D;
    const float* arow = dec + (long long)h * D;
    const float* vrow = vc + (long long)h * E + blockIdx.x * SCAN_COLS;

    auto fetch = [&](int base, int buf) {
        const int n = min(TT, t1 - base);
        if (VEC) {
            for (int tt = 0; tt < n; ++tt) {
                const long long t = base + tt;
#pragma unroll
                for (int sl = 0; sl < NSL; ++sl) {
                    const int d = my_d[sl];
                    if (my_arr[sl] == 0) cp_async16(&sq[buf][tt][d], qrow + t * G * D + d);
                    else if (my_arr[sl] == 1) cp_async16(&sk[buf][tt][d], krow + t * G * D + d);
                    else if (my_arr[sl] == 2) cp_async16(&sa[buf][tt][d], arow + t * H * D + d);
                    else if (GEN && my_arr[sl] == 3) cp_async16(&sr[GEN ? buf : 0][GEN ? tt : 0][d], rem + (t * G + g) * D + d);
                    else if (GEN && my_arr[sl] == 4) cp_async16(&sw[GEN ? buf : 0][GEN ? tt : 0][d], kraw + (t * G + g) * D + d);
                }
            }
            if (tid < n * (SCAN_COLS / 4)) {
                const int tt = tid / (SCAN_COLS / 4), c = (tid % (SCAN_COLS / 4)) * 4;
                if (blockIdx.x * SCAN_COLS + c < E) cp_async16(&sv[buf][tt][c], vrow + (long long)(base + tt) * H * E + c);
            }
            if (!GEN && tid >= 64 && tid < 64 + n) cp_async4(&sb[buf][tid - 64], beta + (long long)(base + tid - 64) * H + h);
            asm volatile("cp.async.commit_group;" ::: "memory");
            return;
        }
        for (int idx = tid; idx < n * D; idx += blockDim.x) {
            const int tt = idx / D, d = idx % D;
            const long long t = base + tt;
            cp_async4(&sq[buf][tt][d], qn + (t * G + g) * D + d);
            cp_async4(&sk[buf][tt][d], kn + (t * G + g) * D + d);
            cp_async4(&sa[buf][tt][d], dec + (t * H + h) * D + d);
            if (GEN) {
                cp_async4(&sr[GEN ? buf : 0][GEN ? tt : 0][d], rem + (t * G + g) * D + d);
                cp_async4(&sw[GEN ? buf : 0][GEN ? tt : 0][d], kraw + (t * G + g) * D + d);
            }
        }
        for (int idx = tid; idx < n * SCAN_COLS; idx += blockDim.x) {
            const int tt = idx / SCAN_COLS, c = idx % SCAN_COLS;
            const int jj = blockIdx.x * SCAN_COLS + c;
            if (jj < E) cp_async4(&sv[buf][tt][c], vc + ((long long)(base + tt) * H + h) * E + jj);
        }
        if (!GEN && tid < n) cp_async4(&sb[buf][tid], beta + (long long)(base + tid) * H + h);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    fetch(t0, 0);
    int buf = 0;
    for (int base = t0; base < t1; base += TT, buf ^= 1) {
        const int n = min(TT, t1 - base);
        if (base + TT < t1) {
            fetch(base + TT, buf ^ 1);                    // (that buffer's readers passed the barrier at the end of the last round)
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        auto token = [&](int tt) {
            const float4* a4 = reinterpret_cast<const float4*>(sa[buf][tt]);
            const float4* k4 = reinterpret_cast<const float4*>(sk[buf][tt]);
            const float4* q4 = reinterpret_cast<const float4*>(sq[buf][tt]);
            if constexpr (GEN) {
                const float4* r4 = reinterpret_cast<const float4*>(sr[buf][tt]);
                const float4* w4 = reinterpret_cast<const float4*>(sw[buf][tt]);
                float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int c = 0; c < NC; ++c) {                     // c = S_old^T u
                    const float4 u4 = k4[c * SCAN_LANES + p];
                    part[0] = fmaf(s[4 * c + 0], u4.x, part[0]);
                    part[1] = fmaf(s[4 * c + 1], u4.y, part[1]);
                    part[2] = fmaf(s[4 * c + 2], u4.z, part[2]);
                    part[3] = fmaf(s[4 * c + 3], u4.w, part[3]);
                }
                float dot = (part[0] + part[1]) + (part[2] + part[3]);
#pragma unroll
                for (int w = 1; w < SCAN_LANES; w <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, w);
                const float v = sv[buf][tt][col];
                float op[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    const float4 a = a4[c * SCAN_LANES + p], rm = r4[c * SCAN_LANES + p], kw = w4[c * SCAN_LANES + p];
                    const float4 q = q4[c * SCAN_LANES + p];
                    s[4 * c + 0] = fmaf(kw.x, v, fmaf(-rm.x, dot, a.x * s[4 * c + 0]));
                    s[4 * c + 1] = fmaf(kw.y, v, fmaf(-rm.y, dot, a.y * s[4 * c + 1]));
                    s[4 * c + 2] = fmaf(kw.z, v, fmaf(-rm.z, dot, a.z * s[4 * c + 2]));
                    s[4 * c + 3] = fmaf(kw.w, v, fmaf(-rm.w, dot, a.w * s[4 * c + 3]));
                    op[0] = fmaf(s[4 * c + 0], q.x, op[0]);
                    op[1] = fmaf(s[4 * c + 1], q.y, op[1]);
                    op[2] = fmaf(s[4 * c + 2], q.z, op[2]);
                    op[3] = fmaf(s[4 * c + 3], q.w, op[3]);
                }
                so[tt][p * SCAN_COLS + col] = (op[0] + op[1]) + (op[2] + op[3]);
                return;
            }
            float4 kk[NC];
            float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const float4 a = a4[c * SCAN_LANES + p];
                kk[c] = k4[c * SCAN_LANES + p];
                s[4 * c + 0] *= a.x; s[4 * c + 1] *= a.y; s[4 * c + 2] *= a.z; s[4 * c + 3] *= a.w;
                part[0] = fmaf(s[4 * c + 0], kk[c].x, part[0]);
                part[1] = fmaf(s[4 * c + 1], kk[c].y, part[1]);
                part[2] = fmaf(s[4 * c + 2], kk[c].z, part[2]);
                part[3] = fmaf(s[4 * c + 3], kk[c].w, part[3]);
            }
            float dot = (part[0] + part[1]) + (part[2] + part[3]);
#pragma unroll
            for (int w = 1; w < SCAN_LANES; w <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, w);
            const float u = sb[buf][tt] * (sv[buf][tt][col] - dot);
            float op[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const float4 q = q4[c * SCAN_LANES + p];
                s[4 * c + 0] = fmaf(kk[c].x, u, s[4 * c + 0]);
                s[4 * c + 1] = fmaf(kk[c].y, u, s[4 * c + 1]);
                s[4 * c + 2] = fmaf(kk[c].z, u, s[4 * c + 2]);
                s[4 * c + 3] = fmaf(kk[c].w, u, s[4 * c + 3]);
                op[0] = fmaf(s[4 * c + 0], q.x, op[0]);
                op[1] = fmaf(s[4 * c + 1], q.y, op[1]);
                op[2] = fmaf(s[4 * c + 2], q.z, op[2]);
                op[3] = fmaf(s[4 * c + 3], q.w, op[3]);
            }
            so[tt][p * SCAN_COLS + col] = (op[0] + op[1]) + (op[2] + op[3]);      // summed over the lanes behind the loop
        };
        if (n == TT) {
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) token(tt);
        } else {
            for (int tt = 0; tt < n; ++tt) token(tt);
        }
        __syncthreads();
        if (tid < n * SCAN_COLS) {                            // one thread a (token, column): the lanes' partial sums in lane order
            const int tt = tid / SCAN_COLS, c = tid % SCAN_COLS;
            const int jj = blockIdx.x * SCAN_COLS + c;
            float o = 0.f;
#pragma unroll
            for (int l = 0; l < SCAN_LANES; ++l) o += so[tt][l * SCAN_COLS + c];
            if (jj < E) out[((long long)(base + tt) * H + h) * E + jj] = o;
        }
        __syncthreads();                                  // this buffer is asked for again in the next round
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int d = ((i >> 2) * SCAN_LANES + p) * 4 + (i & 3);
        if (d < D && j < E) Sh[(long long)d * E + j] = s[i];
    }
}

// One warp a (token, head): o / rms(o) * w * gate(z), z the gate's sums: H * E columns of rows ``ldz`` apart, the sum
// of ``n_parts`` parts; gate: sigmoid(z), or (``silu_gate``) z * sigmoid(z).
template <typename TO>
__global__ void __launch_bounds__(128)
delta_finish_kernel(const float* __restrict__ o, const float* __restrict__ z, long long ldz, int n_parts, long long part_stride,
                    int silu_gate, const float* __restrict__ w, TO* __restrict__ out, int n_tokens, int H, int E, float eps,
                    int w_heads) {
    pdl_trigger();
    pdl_wait();
    const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)n_tokens * H) return;
    const long long t = wid / H;
    const int h = (int)(wid % H);
    const float* orow = o + (t * H + h) * E;
    float ss = 0.f;
    for (int e = lane; e < E; e += 32) { const float v = orow[e]; ss += v * v; }
    ss = warp_sum(ss);
    const float inv = inv_rms(ss, (float)E, eps);
    const float* zrow = z + t * ldz + (long long)h * E;
    if (w_heads) w += (long long)h * E;                   // a weight for every head instead of one shared by the heads
    for (int e = lane; e < E; e += 32) {
        float zv = 0.f;
        for (int i = 0; i < n_parts; ++i) zv += zrow[i * part_stride + e];
        const float g = silu_gate ? zv * sigmoidf_(zv) : sigmoidf_(zv);
        out[(t * H + h) * E + e] = from_f32<TO>(orow[e] * inv * w[e] * g);
    }
}

// The generalised delta rule's inputs, one warp a (token, head).  A projection row holds r, k, v (H heads of D) and the
// removal rate's sums at their columns; ``wpre`` [T, H * D] holds the decay's sums (the low-rank product's result).
//   u = k / sqrt(sum k^2 + unit_eps);  rem = sigmoid(a + a_bias) * u;  w = exp(-decay_scale * sigmoid(wpre + w0))
// r, u, raw k, rem, w and v go out as [T, H * D] float32 each, the scan's operands.
__global__ void __launch_bounds__(128)
gdelta_prepare_kernel(const float* __restrict__ p, long long ldp, int n_parts, long long part_stride, int r_off, int k_off,
                      int v_off, int a_off, const float* __restrict__ a_bias, const float* __restrict__ wpre,
                      const float* __restrict__ w0, float* __restrict__ rn, float* __restrict__ un, float* __restrict__ kraw,
                      float* __restrict__ rem, float* __restrict__ dec, float* __restrict__ vc, int n_tokens, int H, int D,
                      float unit_eps, float decay_scale) {
    pdl_trigger();
    pdl_wait();
    const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)n_tokens * H) return;
    const long long t = wid / H;
    const int h = (int)(wid % H);
    auto at = [&](int c) -> float {
        float v = 0.f;
        for (int i = 0; i < n_parts; ++i) v += p[i * part_stride + t * ldp + c];
        return v;
    };
    float kv[8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int d = lane + 32 * i;
        kv[i] = d < D ? at(k_off + h * D + d) : 0.f;
        ss += kv[i] * kv[i];
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss + unit_eps);
    const long long base = (t * H + h) * D;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int d = lane + 32 * i;
        if (d >= D) continue;
        const int c = h * D + d;
        const float u = kv[i] * inv;
        un[base + d] = u;
        kraw[base + d] = kv[i];
        rem[base + d] = sigmoidf_(at(a_off + c) + a_bias[c]) * u;
        dec[base + d] = expf(-decay_scale * sigmoidf_(wpre[base + d] + w0[c]));
        rn[base + d] = at(r_off + c);
        vc[base + d] = at(v_off + c);
    }
}

UB_API int ub_gdelta_prepare(const float* p, long long ldp, int n_parts, long long part_stride, int r_off, int k_off, int v_off,
                             int a_off, const float* a_bias, const float* wpre, const float* w0, float* rn, float* un,
                             float* kraw, float* rem, float* dec, float* vc, int n_tokens, int H, int D, float unit_eps,
                             float decay_scale, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (H <= 0 || D <= 0 || D > 256 || n_parts < 1) return UB_ERR_ARG;
    const long long warps = (long long)n_tokens * H;
    return (int)ub_launch_dependent(gdelta_prepare_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, st, p, ldp, n_parts,
                                    part_stride, r_off, k_off, v_off, a_off, a_bias, wpre, w0, rn, un, kraw, rem, dec, vc,
                                    n_tokens, H, D, unit_eps, decay_scale);
}

// ---------------------------------------------------------------------------------------
// shape: [H, G, D, E, taps, q_off, k_off, v_off, b_off, a_off] (10 ints)
static int read_shape(const int* shape, long long ldp, int n_parts, long long part_stride, DeltaShape& s) {
    s.H = shape[0]; s.G = shape[1]; s.D = shape[2]; s.E = shape[3]; s.taps = shape[4];
    s.q_off = shape[5]; s.k_off = shape[6]; s.v_off = shape[7]; s.b_off = shape[8]; s.a_off = shape[9];
    s.ldp = ldp; s.n_parts = n_parts; s.part_stride = part_stride;
    if (s.H <= 0 || s.G <= 0 || s.H % s.G || s.D <= 0 || s.D > 256 || s.E <= 0 || s.taps < 1 || s.taps > MAX_TAPS ||
        s.H > 65535 || n_parts < 1) return UB_ERR_ARG;
    // the convolution's state is indexed by projection column: q, k, v are the row's first columns
    if (s.q_off != 0 || s.k_off != s.G * s.D || s.v_off != 2 * s.G * s.D) return UB_ERR_ARG;
    return 0;
}

UB_API int ub_delta_prepare(const float* p, long long ldp, int n_parts, long long part_stride, const int* shape,
                            const float* conv_w, float* conv_state, int update_state, const float* dpre,
                            const float* dt_bias, const float* a_log, const int* tok_seq,
                            const int* seq_start, const int* seq_slot, float* qn, float* kn, float* vc, float* beta,
                            float* dec, int n_tokens, float unit_eps, float q_scale, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    DeltaShape s;
    if (int rc = read_shape(shape, ldp, n_parts, part_stride, s)) return rc;
    const long long warps = (long long)n_tokens * (2 * s.G + s.H);
    const unsigned grid = (unsigned)((warps + 3) / 4);
    return (int)ub_launch_dependent(delta_prepare_kernel, dim3(grid), dim3(128), 0, st, p, s, conv_w, conv_state, update_state, dpre, dt_bias,
                                    a_log, tok_seq, seq_start, seq_slot, qn, kn, vc, beta, dec, n_tokens, unit_eps, q_scale);
}

UB_API int ub_conv_state_update(const float* p, long long ldp, int n_parts, long long part_stride, float* conv_state,
                                const int* seq_start, const int* seq_slot, int n_seqs, int C, int taps, cudaStream_t st) {
    if (n_seqs <= 0 || taps <= 1) return 0;
    if (taps > MAX_TAPS || n_parts < 1) return UB_ERR_ARG;
    DeltaShape s = {};
    s.ldp = ldp; s.n_parts = n_parts; s.part_stride = part_stride;
    const long long n = (long long)n_seqs * C;
    return (int)ub_launch_dependent(conv_state_update_kernel, dim3((unsigned)((n + 127) / 128)), dim3(128), 0, st, p, s,
                                    conv_state, seq_start, seq_slot, n_seqs, C, taps);
}

UB_API int ub_delta_scan(const float* qn, const float* kn, const float* vc, const float* beta, const float* dec, float* out,
                         float* S, const int* seq_start, const int* seq_slot, int n_seqs, int n_tokens, int H, int G, int D,
                         int E, int sm_count, const float* rem, const float* kraw, cudaStream_t st) {
    if (n_seqs <= 0) return 0;
    const bool gen = rem != nullptr;
    if (gen != (kraw != nullptr)) return UB_ERR_ARG;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || D > 256 || E <= 0 || H > 65535 || n_seqs > 65535) return UB_ERR_ARG;
    const bool vec = D % 4 == 0 && E % 4 == 0 &&
        (((uintptr_t)qn | (uintptr_t)kn | (uintptr_t)vc | (uintptr_t)dec | (uintptr_t)rem | (uintptr_t)kraw) & 15) == 0;
    // lanes a column: eight, and more (fewer values and a shorter chain a thread) only while the launch still has
    // no more than about one warp for every scheduler and every lane gets a whole float4 chunk; measured at 2,048
    // tokens, 16 heads, sizes of 128: 346 / 372 / 405 ns a token with 8 / 16 / 32 lanes, at sizes of 64: 322 / 296
    static const int forced = getenv("ULTIMA_SCAN_LANES") ? atoi(getenv("ULTIMA_SCAN_LANES")) : 0;    // for measurements
    const long long budget = 4LL * (sm_count > 0 ? sm_count : 148);
    auto warps_with = [&](int l) { return (long long)n_seqs * H * ((E * l + 127) / 128) * 4; };
    int lanes = 8;
    while (lanes < 32 && lanes * 2 * 4 <= ((D + 3) / 4) * 4 && warps_with(lanes * 2) <= budget) lanes <<= 1;
    if (forced == 8 || forced == 16 || forced == 32) lanes = forced;
    while (lanes > 8 && lanes * 4 > ((D + 3) / 4) * 4) lanes >>= 1;
    const int cols = 128 / lanes;
    const dim3 grid((E + cols - 1) / cols, H, n_seqs), block(128);
    const int per_lane = (D + lanes - 1) / lanes;          // key channels a lane, rounded up to whole chunks
    const int R = per_lane <= 4 ? 4 : per_lane <= 8 ? 8 : per_lane <= 16 ? 16 : 32;
    cudaError_t e = cudaErrorInvalidValue;
    // A step that brings more than one token a sequence starts as an ordinary launch, behind the end of the kernels before
    // it.  As a programmatic dependent its few CTAs (one for an SM or fewer, each busy for the whole step) are placed while
    // the kernel before drains, on the SMs that happen to have room first, several to an SM: measured, a prompt of 2,048
    // tokens with four such layers took 8.2 ms so and 6.6 ms with every CTA on an SM of its own.
    const bool dep = n_tokens <= n_seqs;
#define GO2(RR, LL, VV, GG) ub_launch_ordered(dep, delta_scan_kernel<RR, LL, VV, GG>, grid, block, 0, st, qn, kn, vc, beta, dec, out, S, seq_start, seq_slot, H, G, D, E, rem, kraw)
#define GO(RR, LL) e = gen ? (vec ? GO2(RR, LL, true, true) : GO2(RR, LL, false, true)) : (vec ? GO2(RR, LL, true, false) : GO2(RR, LL, false, false))
    if (lanes == 32) { if (R == 4) GO(4, 32); else if (R == 8) GO(8, 32); else return UB_ERR_ARG; }
    else if (lanes == 16) { if (R == 4) GO(4, 16); else if (R == 8) GO(8, 16); else if (R == 16) GO(16, 16); else return UB_ERR_ARG; }
    else { if (R == 4) GO(4, 8); else if (R == 8) GO(8, 8); else if (R == 16) GO(16, 8); else GO(32, 8); }
#undef GO
#undef GO2
    return (int)e;
}

UB_API int ub_delta_finish(const float* o, const float* z, long long ldz, int n_parts, long long part_stride, int silu_gate,
                           const float* w, void* out, int out_dtype, int n_tokens, int H, int E, float eps, int w_heads,
                           cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (n_parts < 1) return UB_ERR_ARG;
    const long long warps = (long long)n_tokens * H;
    const unsigned grid = (unsigned)((warps + 3) / 4);
    cudaError_t e;
    if (out_dtype == UB_F32)
        e = ub_launch_dependent(delta_finish_kernel<float>, dim3(grid), dim3(128), 0, st, o, z, ldz, n_parts, part_stride, silu_gate, w, (float*)out, n_tokens, H, E, eps, w_heads);
    else if (out_dtype == UB_BF16)
        e = ub_launch_dependent(delta_finish_kernel<__nv_bfloat16>, dim3(grid), dim3(128), 0, st, o, z, ldz, n_parts, part_stride, silu_gate, w, (__nv_bfloat16*)out, n_tokens, H, E, eps, w_heads);
    else return UB_ERR_UNSUPPORTED;
    return (int)e;
}
