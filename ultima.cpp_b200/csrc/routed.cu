// A routed feed-forward (mixture of experts): which experts a token uses, the order its rows are worked in,
// and the weighted sum of what the experts return.  The experts' products themselves are grouped matrix
// products over the sorted rows (gemm_simt.cu; gemm_tcgen05.cu for bfloat16).
//
//   route     one warp a token: s = softmax(z) over all router outputs (float32); choice scores s + correction;
//             with groups, only the outputs of the ``keep`` groups with the largest choice score stay (the
//             others count as -inf); the ``top`` largest choice scores are chosen, lowest index first among
//             equals; a chosen output's weight is its s (no renormalisation).  Outputs from ``n_experts`` on
//             are identity experts.  Counts the rows of every real expert.
//   plan      one block: the experts' segments of the sorted rows (first row of each), the tiles of up to
//             ``tile`` rows (expert, first row, rows) that the grouped products run over, their number; clears
//             the counters for the next use.
//   scatter   one thread a (token, choice): its place in its expert's segment (``row_pos``; -1 for an identity
//             expert) and, for that place, the token it is (``src_rows``).
//   gather    one block a (token, choice): the token's input row is copied to its sorted place, for a grouped
//             product that reads its rows in the sorted order (the tensor-core one: a tile is one TMA box).
//   combine   one block a token: residual += sum_k w_k * (expert row k, or the token's own input for an
//             identity expert), in the order of k.
// ``mode`` (bits) and ``wscale`` choose another router of the same family: bit 0, s = sigmoid(z) instead of the softmax;
// bit 1, a group's score is the sum of its two largest choice scores instead of the largest; bit 2, the chosen outputs'
// weights are divided by their sum (+ 1e-20); the weights are then multiplied by ``wscale``.
// Places within a segment are handed out by an atomic counter, so they differ from run to run; every row of a
// product is computed on its own, so no result depends on them.
#include "common.cuh"

constexpr int ROUTE_WARPS = 4;

// One token's routing by one warp: zr its logits (``n_parts`` slices ``part_stride`` apart), sc / ch / gm the warp's
// work space ([n_out], [n_out], [n_groups]), idx_t / wts_t the token's ``top`` results, counts the experts' row counters
// (global or shared memory).
__device__ __forceinline__ void route_token(const float* __restrict__ zr, int n_parts, long long part_stride,
                                            const float* __restrict__ corr, int n_out, int n_experts, int top, int n_groups,
                                            int keep, float* sc, float* ch, float* gm, int lane, int* idx_t, float* wts_t,
                                            int* counts, int mode, float wscale) {
    float m = -INFINITY;
    for (int i = lane; i < n_out; i += 32) {              // the logits may come as K slices: summed in the slices' order
        float v = zr[i];
        for (int s = 1; s < n_parts; ++s) v += zr[s * part_stride + i];
        sc[i] = v;
        m = fmaxf(m, v);
    }
    if (mode & 1) {
        for (int i = lane; i < n_out; i += 32) { const float s = 1.0f / (1.0f + expf(-sc[i])); sc[i] = s; ch[i] = s + (corr ? corr[i] : 0.f); }
    } else {
        m = warp_max(m);
        float sum = 0.f;
        for (int i = lane; i < n_out; i += 32) { const float e = expf(sc[i] - m); sc[i] = e; sum += e; }
        sum = warp_sum(sum);
        for (int i = lane; i < n_out; i += 32) { const float s = sc[i] / sum; sc[i] = s; ch[i] = s + (corr ? corr[i] : 0.f); }
    }
    __syncwarp();
    if (n_groups > 1 && keep < n_groups) {
        const int size = n_out / n_groups;
        for (int g = lane; g < n_groups; g += 32) {
            float b = -INFINITY, b2 = -INFINITY;           // the largest and the second largest
            for (int i = 0; i < size; ++i) {
                const float v = ch[g * size + i];
                if (v > b) { b2 = b; b = v; } else if (v > b2) b2 = v;
            }
            gm[g] = ((mode & 2) && size > 1) ? b + b2 : b;
        }
        __syncwarp();
        // the kept groups are marked with +inf; what is left unmarked loses its outputs
        for (int r = 0; r < keep; ++r) {
            float best = -INFINITY;
            int at = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32) {
                const float v = gm[g];
                if (v != INFINITY && (v > best || (v == best && g < at))) { best = v; at = g; }
            }
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
            }
            if (lane == 0 && at != 0x7fffffff) gm[at] = INFINITY;
            __syncwarp();
        }
        for (int i = lane; i < n_out; i += 32)
            if (gm[i / size] != INFINITY) ch[i] = -INFINITY;
        __syncwarp();
    }
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int i = lane; i < n_out; i += 32) {
            const float v = ch[i];
            if (!isnan(v) && (v > best || (v == best && i < at))) { best = v; at = i; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at == 0x7fffffff) at = 0;                     // (every score was taken or not a number: a row of NaN)
        if (lane == 0) {
            idx_t[k] = at;
            wts_t[k] = sc[at];
            ch[at] = NAN;                                 // taken: NaN is passed over, while -inf may still be chosen
            if (at < n_experts) atomicAdd(&counts[at], 1);
        }
        __syncwarp();
    }
    if (lane == 0 && ((mode & 4) || wscale != 1.0f)) {
        float f = wscale;
        if (mode & 4) {
            float sum = 0.f;
            for (int k = 0; k < top; ++k) sum += wts_t[k];
            f = wscale / (sum + 1e-20f);
        }
        for (int k = 0; k < top; ++k) wts_t[k] *= f;
    }
}

__global__ void __launch_bounds__(ROUTE_WARPS * 32)
route_kernel(const float* __restrict__ z, long long ldz, int n_parts, long long part_stride, const float* __restrict__ corr,
             int n_tokens, int n_out, int n_experts, int top, int n_groups, int keep, int* __restrict__ idx,
             float* __restrict__ wts, int* __restrict__ counts, int mode, float wscale) {
    extern __shared__ float sm[];
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long t = (long long)blockIdx.x * ROUTE_WARPS + warp;
    if (t >= n_tokens) return;
    float* sc = sm + (size_t)warp * (2 * n_out + n_groups);      // scores
    float* ch = sc + n_out;                                      // choice scores
    float* gm = ch + n_out;                                      // a group's best choice score
    route_token(z + t * ldz, n_parts, part_stride, corr, n_out, n_experts, top, n_groups, keep, sc, ch, gm, lane,
                idx + t * top, wts + t * top, counts, mode, wscale);
}

// route, plan and scatter of a step of few tokens in ONE block (the counters live in shared memory; the global ones are
// not touched and stay zero): three launches of a decode step become one.
constexpr int SMALL_WARPS = 16;          // a token a warp: more tokens than warps and the separate kernels are faster

__global__ void __launch_bounds__(SMALL_WARPS * 32)
route_small_kernel(const float* __restrict__ z, long long ldz, int n_parts, long long part_stride, const float* __restrict__ corr,
                   int n_tokens, int n_out, int n_experts, int top, int n_groups, int keep, int* __restrict__ idx,
                   float* __restrict__ wts, int4* __restrict__ tiles, int* __restrict__ n_tiles, int* __restrict__ row_pos,
                   int* __restrict__ src_rows, int tile, int mode, float wscale) {
    extern __shared__ float sm[];
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_warp = 2 * n_out + n_groups;
    int* cnt = (int*)(sm + (size_t)SMALL_WARPS * per_warp);     // [n_experts] rows of every expert
    int* cursor = cnt + n_experts;                              // [n_experts] places handed out
    int* seg = cursor + n_experts;                              // [n_experts] first sorted row
    int* first_tile = seg + n_experts;                          // [n_experts + 1]
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) { cnt[e] = 0; cursor[e] = 0; }
    __syncthreads();
    float* sc = sm + (size_t)warp * per_warp;
    for (int t = warp; t < n_tokens; t += SMALL_WARPS) {
        route_token(z + (long long)t * ldz, n_parts, part_stride, corr, n_out, n_experts, top, n_groups, keep, sc, sc + n_out,
                    sc + 2 * n_out, lane, idx + (long long)t * top, wts + (long long)t * top, cnt, mode, wscale);
        __syncwarp();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int row = 0, tl = 0;
        for (int e = 0; e < n_experts; ++e) {
            seg[e] = row;
            first_tile[e] = tl;
            row += cnt[e];
            tl += (cnt[e] + tile - 1) / tile;
        }
        first_tile[n_experts] = tl;
        *n_tiles = tl;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        const int n = cnt[e], r0 = seg[e];
        for (int i = 0; i * tile < n; ++i) tiles[first_tile[e] + i] = make_int4(e, r0 + i * tile, min(tile, n - i * tile), 0);
    }
    for (int i = threadIdx.x; i < n_tokens * top; i += blockDim.x) {
        const int e = idx[i];                                   // written by this block before the barriers above
        if (e >= n_experts) { row_pos[i] = -1; continue; }
        const int p = seg[e] + atomicAdd(&cursor[e], 1);
        row_pos[i] = p;
        src_rows[p] = i / top;
    }
}

__global__ void plan_kernel(int* __restrict__ counts, int* __restrict__ cursor, int* __restrict__ seg_start,
                            int4* __restrict__ tiles, int* __restrict__ n_tiles, int n_experts, int tile) {
    extern __shared__ int sh[];          // [n_experts] counts, [n_experts + 1] first tile of each expert
    pdl_trigger();
    pdl_wait();
    int* cnt = sh;
    int* first_tile = sh + n_experts;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) { cnt[e] = counts[e]; counts[e] = 0; cursor[e] = 0; }
    __syncthreads();
    if (threadIdx.x == 0) {
        int row = 0, tl = 0;
        for (int e = 0; e < n_experts; ++e) {
            seg_start[e] = row;
            first_tile[e] = tl;
            row += cnt[e];
            tl += (cnt[e] + tile - 1) / tile;
        }
        first_tile[n_experts] = tl;
        *n_tiles = tl;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        const int n = cnt[e], r0 = seg_start[e];
        for (int i = 0; i * tile < n; ++i) tiles[first_tile[e] + i] = make_int4(e, r0 + i * tile, min(tile, n - i * tile), 0);
    }
}

__global__ void scatter_kernel(const int* __restrict__ idx, const int* __restrict__ seg_start, int* __restrict__ cursor,
                               int* __restrict__ row_pos, int* __restrict__ src_rows, long long n, int top, int n_experts) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int e = idx[i];
    if (e >= n_experts) { row_pos[i] = -1; return; }
    const int p = seg_start[e] + atomicAdd(&cursor[e], 1);
    row_pos[i] = p;
    src_rows[p] = (int)(i / top);
}

__global__ void gather_kernel(const uint4* __restrict__ h, const int* __restrict__ row_pos, uint4* __restrict__ sorted,
                              int top, int row_vecs) {
    pdl_trigger();
    pdl_wait();
    const int p = row_pos[blockIdx.x];
    if (p < 0) return;
    const uint4* src = h + (long long)(blockIdx.x / top) * row_vecs;
    uint4* dst = sorted + (long long)p * row_vecs;
    for (int c = threadIdx.x; c < row_vecs; c += blockDim.x) dst[c] = src[c];
}

template <typename TH, typename TY>
__global__ void combine_kernel(const TY* __restrict__ y, const TH* __restrict__ h, const int* __restrict__ row_pos,
                               const float* __restrict__ wts, float* __restrict__ residual, int width, int top) {
    pdl_trigger();
    pdl_wait();
    const long long t = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int p = row_pos[t * top + k];
            const float v = p >= 0 ? to_f32<TY>(y[(long long)p * width + c]) : to_f32<TH>(h[t * width + c]);
            acc = fmaf(wts[t * top + k], v, acc);
        }
        residual[t * width + c] += acc;
    }
}

// The same sum four columns a thread and a part of a row a block (width a multiple of 4, rows 16-byte aligned): a step
// of few tokens still fills the SMs.  An element's sum has the order of the kernel above.
template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

template <typename TH, typename TY>
__global__ void combine_vec_kernel(const TY* __restrict__ y, const TH* __restrict__ h, const int* __restrict__ row_pos,
                                   const float* __restrict__ wts, float* __restrict__ residual, int width, int top) {
    pdl_trigger();
    pdl_wait();
    const long long t = blockIdx.x;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (c >= width) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < top; ++k) {
        const int p = row_pos[t * top + k];
        const float w = wts[t * top + k];
        const float4 v = p >= 0 ? load4<TY>(y + (long long)p * width + c) : load4<TH>(h + t * width + c);
        acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y); acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
    }
    float4* r = reinterpret_cast<float4*>(residual + t * width + c);
    float4 o = *r;
    o.x += acc.x; o.y += acc.y; o.z += acc.z; o.w += acc.w;
    *r = o;
}

// z: the router's logits [tokens, outputs] (row stride ldz), or ``n_parts`` such arrays ``part_stride`` floats apart
// whose sum they are.
UB_API int ub_route(const float* z, long long ldz, int n_parts, long long part_stride, const float* corr, int n_tokens,
                    int n_out, int n_experts, int top, int n_groups, int keep, int* idx, float* wts, int* counts,
                    int mode, float wscale, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (n_parts < 1) return UB_ERR_ARG;
    if (n_out < 1 || n_experts < 0 || n_experts > n_out || top < 1 || top > n_out || n_groups < 1 || n_out % n_groups ||
        keep < 1 || keep > n_groups) return UB_ERR_ARG;
    const size_t smem = (size_t)ROUTE_WARPS * (2 * n_out + n_groups) * sizeof(float);
    if (smem > 48 * 1024) return UB_ERR_ARG;
    const unsigned grid = (unsigned)((n_tokens + ROUTE_WARPS - 1) / ROUTE_WARPS);
    return (int)ub_launch_dependent(route_kernel, dim3(grid), dim3(ROUTE_WARPS * 32), smem, st, z, ldz, n_parts, part_stride, corr,
                                    n_tokens, n_out, n_experts, top, n_groups, keep, idx, wts, counts, mode, wscale);
}

// The three steps above in one launch, for steps of at most ROUTE_SMALL_TOKENS tokens.
constexpr int ROUTE_SMALL_TOKENS = SMALL_WARPS;
UB_API int ub_route_small_tokens() { return ROUTE_SMALL_TOKENS; }

UB_API int ub_route_small(const float* z, long long ldz, int n_parts, long long part_stride, const float* corr, int n_tokens,
                          int n_out, int n_experts, int top, int n_groups, int keep, int* idx, float* wts, void* tiles,
                          int* n_tiles, int* row_pos, int* src_rows, int tile, int mode, float wscale, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (n_parts < 1 || n_tokens > ROUTE_SMALL_TOKENS || tile < 1) return UB_ERR_ARG;
    if (n_out < 1 || n_experts < 1 || n_experts > n_out || top < 1 || top > n_out || n_groups < 1 || n_out % n_groups ||
        keep < 1 || keep > n_groups) return UB_ERR_ARG;
    const size_t smem = (size_t)SMALL_WARPS * (2 * n_out + n_groups) * sizeof(float) + (size_t)(4 * n_experts + 1) * sizeof(int);
    if (smem > 48 * 1024) return UB_ERR_ARG;
    return (int)ub_launch_dependent(route_small_kernel, dim3(1), dim3(SMALL_WARPS * 32), smem, st, z, ldz, n_parts, part_stride,
                                    corr, n_tokens, n_out, n_experts, top, n_groups, keep, idx, wts, (int4*)tiles, n_tiles,
                                    row_pos, src_rows, tile, mode, wscale);
}

UB_API int ub_route_plan(int* counts, int* cursor, int* seg_start, void* tiles, int* n_tiles, int n_experts, int tile,
                         cudaStream_t st) {
    if (n_experts < 1 || tile < 1) return UB_ERR_ARG;
    const size_t smem = (size_t)(2 * n_experts + 1) * sizeof(int);
    if (smem > 48 * 1024) return UB_ERR_ARG;
    return (int)ub_launch_dependent(plan_kernel, dim3(1), dim3(256), smem, st, counts, cursor, seg_start, (int4*)tiles, n_tiles,
                                    n_experts, tile);
}

UB_API int ub_route_scatter(const int* idx, const int* seg_start, int* cursor, int* row_pos, int* src_rows, int n_tokens,
                            int top, int n_experts, cudaStream_t st) {
    const long long n = (long long)n_tokens * top;
    if (n <= 0) return 0;
    return (int)ub_launch_dependent(scatter_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, idx, seg_start, cursor,
                                    row_pos, src_rows, n, top, n_experts);
}

// y: the experts' results for the sorted rows [rows, width] (float32 or bfloat16); h: the feed-forward's input
// [tokens, width], which an identity expert hands on.
UB_API int ub_route_combine(const void* y, int y_dtype, const void* h, int h_dtype, const int* row_pos, const float* wts,
                            float* residual, int n_tokens, int width, int top, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    const int threads = width >= 1024 ? 256 : 128;
    cudaError_t e;
    const bool vec = width % 4 == 0 && !(((uintptr_t)y | (uintptr_t)h | (uintptr_t)residual) & 15);
    const int vthreads = 128;
    const dim3 vgrid(n_tokens, (width / 4 + vthreads - 1) / vthreads);
#define GO(TH, TY) e = vec ? ub_launch_dependent(combine_vec_kernel<TH, TY>, vgrid, dim3(vthreads), 0, st, (const TY*)y, (const TH*)h, \
                                                 row_pos, wts, residual, width, top) \
                           : ub_launch_dependent(combine_kernel<TH, TY>, dim3(n_tokens), dim3(threads), 0, st, (const TY*)y, (const TH*)h, \
                                                 row_pos, wts, residual, width, top)
    if (h_dtype == UB_F32 && y_dtype == UB_F32) GO(float, float);
    else if (h_dtype == UB_BF16 && y_dtype == UB_F32) GO(__nv_bfloat16, float);
    else if (h_dtype == UB_BF16 && y_dtype == UB_BF16) GO(__nv_bfloat16, __nv_bfloat16);
    else return UB_ERR_UNSUPPORTED;
#undef GO
    return (int)e;
}

// sorted[row_pos[t * top + k]] = h[t] for every choice with a row; rows of ``row_bytes`` bytes (a multiple of 16, both
// buffers 16-byte aligned).
UB_API int ub_route_gather(const void* h, const int* row_pos, void* sorted, int n_tokens, int top, long long row_bytes,
                           cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (top < 1 || row_bytes < 16 || (row_bytes % 16) || ((uintptr_t)h & 15) || ((uintptr_t)sorted & 15)) return UB_ERR_ARG;
    const int vecs = (int)(row_bytes / 16);
    return (int)ub_launch_dependent(gather_kernel, dim3((unsigned)(n_tokens * top)), dim3(vecs < 256 ? ((vecs + 31) / 32) * 32 : 256),
                                    0, st, (const uint4*)h, row_pos, (uint4*)sorted, top, vecs);
}
