// Routing for a feed-forward made of small experts, of which every token uses a few.
//
//   router_gates   logits z = W_router x in 32-bit (spread over blocks by expert; the block of a token that finishes last goes on);
//                  the `top` largest are chosen (the lower index wins a tie) and the
//                  token's weights are the softmax over the chosen logits alone (or, with `over_all`, the chosen
//                  experts' shares of the softmax over ALL logits, which then do not sum to one; or, with rule 2, sigmoid
//                  scores: the choice looks at sigmoid(z) + correction, and only inside the `keep` of `groups` equal
//                  groups of neighbouring experts whose two largest such numbers sum highest, and the weights are
//                  the chosen experts' sigmoid(z) as they are).  The result is the dense matrix
//                  gates [T, experts], zero where an expert was not chosen, plus the chosen ids and weights.
//   relu2_gate     hidden[t, e * ff + j] = relu(up[t, e * ff + j])^2 * gates[t, e]: with the experts' up matrices
//                  stacked along the rows and their down matrices side by side along the columns, the product
//                  hidden W_down^T is the weighted sum of the chosen experts' outputs, and an expert that was not
//                  chosen contributes exact zeros.
//
// Nothing here waits for the host or depends on how many tokens an expert drew, so a step can be captured in a graph.
#include "common.cuh"

#define ROUTER_WARPS 4

// Four values of a row as floats, from 32-bit or bfloat16 storage (16- and 8-byte loads).
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    const float2 a = __bfloat1622float2(lo), b = __bfloat1622float2(hi);
    return make_float4(a.x, a.y, b.x, b.y);
}

// What the block that finishes a token's logits last does with them: warp `warp` of `warps` takes the token's row `out`
// [experts] of logits (read past L1), picks the `top` largest one after the other (the lower index wins a tie) and
// overwrites the row with the routing weights.  `logits_s` [experts] is this warp's shared scratch.
// How the weights come from the logits.  mode 0: softmax over the chosen logits; 1: the chosen experts' shares of the
// softmax over all; 2: sigmoid scores with a correction on the choice and a choice among groups (see the top of the file).
struct RouterRule {
    int mode;
    const float* correction;  // [experts] or null (mode 2)
    int groups, keep;         // mode 2; one group of which one is kept: no limit
};
// Floats of shared scratch a warp needs to choose for one token: logits, scores, group scores.
#define ROUTER_SCRATCH(experts) (3 * (size_t)(experts))

__device__ __forceinline__ void choose_experts(float* __restrict__ out, float* logits_s, int* __restrict__ chosen_ids,
                                               float* __restrict__ chosen_weights, int experts, int top, int lane,
                                               const RouterRule rule) {
    const int over_all = rule.mode == 1;
    const bool scored = rule.mode == 2;
    float* scores_s = logits_s + experts;       // mode 2: sigmoid(z), the weights
    float* groups_s = logits_s + 2 * experts;   // mode 2: every group's two largest choice scores, summed
    for (int i = lane; i < experts; i += 32) logits_s[i] = __ldcg(out + i);
    __syncwarp();
    for (int i = lane; i < experts; i += 32) out[i] = 0.0f;
    __syncwarp();
    if (scored) {
        for (int i = lane; i < experts; i += 32) {
            const float score = 1.0f / (1.0f + expf(-logits_s[i]));
            scores_s[i] = score;
            logits_s[i] = score + (rule.correction ? rule.correction[i] : 0.0f);  // what the choice looks at
        }
        __syncwarp();
        if (rule.groups > 1 && rule.keep < rule.groups) {
            const int size = experts / rule.groups;
            for (int g = lane; g < rule.groups; g += 32) {
                float first = -INFINITY, second = -INFINITY;
                for (int j = 0; j < size; ++j) {
                    const float c = logits_s[g * size + j];
                    if (c > first) second = first, first = c;
                    else if (c > second) second = c;
                }
                groups_s[g] = size > 1 ? first + second : first;
            }
            __syncwarp();
            // a group stays open when fewer than `keep` groups stand ahead of it (the lower index wins a tie)
            for (int g = lane; g < rule.groups; g += 32) {
                const float mine = groups_s[g];
                int ahead = 0;
                for (int o = 0; o < rule.groups; ++o) {
                    const float other = groups_s[o];
                    ahead += (other > mine || (other == mine && o < g)) ? 1 : 0;
                }
                if (ahead >= rule.keep)
                    for (int j = 0; j < size; ++j) logits_s[g * size + j] = -INFINITY;
            }
            __syncwarp();
        }
    }
    float best_first = 0.0f, denom = 0.0f, all_sum = 0.0f;
    if (over_all) {
        // the softmax's denominator over every expert, before any logit is struck out
        float all_max = -INFINITY;
        for (int i = lane; i < experts; i += 32) all_max = fmaxf(all_max, logits_s[i]);
        all_max = warp_max(all_max);
        for (int i = lane; i < experts; i += 32) all_sum += expf(logits_s[i] - all_max);
        all_sum = warp_sum(all_sum);
    }
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int i = lane; i < experts; i += 32) {
            const float z = logits_s[i];
            if (z > best || (z == best && i < best_e)) {
                best = z;
                best_e = i;
            }
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, best, offset);
            const int other_e = __shfl_xor_sync(0xffffffffu, best_e, offset);
            if (other > best || (other == best && other_e < best_e)) {
                best = other;
                best_e = other_e;
            }
        }
        if (best_e == 0x7fffffff) {  // fewer comparable logits than `top` (a row of NaN): the rest stays unchosen
            if (lane == 0 && chosen_ids)
                for (int rest = k; rest < top; ++rest) chosen_ids[rest] = -1, chosen_weights[rest] = 0.0f;
            break;
        }
        if (k == 0) best_first = best;
        const float weight = scored ? scores_s[best_e] : expf(best - best_first);  // the first chosen logit is the largest
        denom += weight;
        if (lane == 0) {
            out[best_e] = weight;
            if (chosen_ids) chosen_ids[k] = best_e, chosen_weights[k] = weight;
            logits_s[best_e] = -INFINITY;
        }
        __syncwarp();
    }
    __syncwarp();
    if (over_all) denom = all_sum;  // (the first chosen logit is the maximum of all)
    const float inv = scored ? 1.0f : (denom > 0.0f ? 1.0f / denom : 0.0f);
    for (int i = lane; i < experts; i += 32) out[i] *= inv;
    if (chosen_weights)
        for (int k = lane; k < top; k += 32) chosen_weights[k] *= inv;
}

// Counts this block in on `counter`; true in the block that arrives last (which sets the counter back to zero for the
// next launch).  Everything the other blocks wrote before their arrival is visible to that block afterwards.
__device__ __forceinline__ bool arrives_last(int* counter, int blocks, int* flag_s) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int before = atomicAdd(counter, 1);
        *flag_s = before == blocks - 1;
        if (*flag_s) *counter = 0;
    }
    __syncthreads();
    const bool last = *flag_s != 0;
    if (last) __threadfence();
    return last;
}

// Few tokens: a block per (token, expert); its four warps take a quarter of the row each, so that a step of a handful of
// tokens spreads over tokens x experts blocks with a few loads per lane.  The last block of a token chooses.
template <typename T>
__global__ void __launch_bounds__(ROUTER_WARPS * 32)
router_gates_few_kernel(const T* __restrict__ x, long x_stride, const float* __restrict__ router, float* __restrict__ gates,
                        int* __restrict__ chosen_ids, float* __restrict__ chosen_weights, int* __restrict__ arrivals, int hidden,
                        int experts, int top, RouterRule rule) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float logits_s[];  // [experts]
    __shared__ float part_s[ROUTER_WARPS];
    __shared__ int is_last;
    const int token = blockIdx.x, e = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* row = x + (size_t)token * x_stride;
    const float* w = router + (size_t)e * hidden;
    float* out = gates + (size_t)token * experts;
    float dot = 0.0f;
    if (hidden % 4 == 0 && x_stride % 4 == 0 && (((uintptr_t)x | (uintptr_t)router) & 15) == 0) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
        for (int i = threadIdx.x * 4; i < hidden; i += ROUTER_WARPS * 128) {
            const float4 a = load4(row + i), b = load4(w + i);
            acc[0] = fmaf(a.x, b.x, acc[0]);
            acc[1] = fmaf(a.y, b.y, acc[1]);
            acc[2] = fmaf(a.z, b.z, acc[2]);
            acc[3] = fmaf(a.w, b.w, acc[3]);
        }
        dot = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    } else {
        for (int i = threadIdx.x; i < hidden; i += ROUTER_WARPS * 32) dot = fmaf(to_f32<T>(row[i]), w[i], dot);
    }
    dot = warp_sum(dot);
    if (lane == 0) part_s[warp] = dot;
    __syncthreads();
    if (threadIdx.x == 0) out[e] = (part_s[0] + part_s[1]) + (part_s[2] + part_s[3]);
    if (!arrives_last(&arrivals[token], (int)gridDim.y, &is_last)) return;
    if (warp == 0)
        choose_experts(out, logits_s, chosen_ids ? chosen_ids + (size_t)token * top : nullptr,
                       chosen_weights ? chosen_weights + (size_t)token * top : nullptr, experts, top, lane, rule);
}

// Many tokens: a block takes ROUTER_TOKENS tokens and ROUTER_WARPS experts, a warp per expert, so that a router row is
// read once for eight tokens (a block per token read the whole router matrix from L2 for every token).  The last block
// of a group of tokens chooses for them, a warp per token in turn.
#define ROUTER_TOKENS 8
template <typename T>
__global__ void __launch_bounds__(ROUTER_WARPS * 32)
router_gates_many_kernel(const T* __restrict__ x, long x_stride, const float* __restrict__ router, float* __restrict__ gates,
                         int* __restrict__ chosen_ids, float* __restrict__ chosen_weights, int* __restrict__ arrivals, int tokens,
                         int hidden, int experts, int top, RouterRule rule) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float logits_s[];  // [ROUTER_WARPS][experts]
    __shared__ int is_last;
    const int first = blockIdx.x * ROUTER_TOKENS;
    const int count = min(ROUTER_TOKENS, tokens - first);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int e = blockIdx.y * ROUTER_WARPS + warp;
    if (e < experts) {
        const float* w = router + (size_t)e * hidden;
        float dot[ROUTER_TOKENS];
#pragma unroll
        for (int t = 0; t < ROUTER_TOKENS; ++t) dot[t] = 0.0f;
        if (hidden % 4 == 0 && x_stride % 4 == 0 && (((uintptr_t)x | (uintptr_t)router) & 15) == 0) {
#pragma unroll 2
            for (int i = lane * 4; i < hidden; i += 128) {
                const float4 b = load4(w + i);
#pragma unroll
                for (int t = 0; t < ROUTER_TOKENS; ++t) {
                    if (t < count) {
                        const float4 a = load4(x + (size_t)(first + t) * x_stride + i);
                        dot[t] = fmaf(a.x, b.x, fmaf(a.y, b.y, fmaf(a.z, b.z, fmaf(a.w, b.w, dot[t]))));
                    }
                }
            }
        } else {
            for (int i = lane; i < hidden; i += 32) {
                const float b = w[i];
#pragma unroll
                for (int t = 0; t < ROUTER_TOKENS; ++t)
                    if (t < count) dot[t] = fmaf(to_f32<T>(x[(size_t)(first + t) * x_stride + i]), b, dot[t]);
            }
        }
#pragma unroll
        for (int t = 0; t < ROUTER_TOKENS; ++t) {
            const float total = warp_sum(dot[t]);
            if (lane == 0 && t < count) gates[(size_t)(first + t) * experts + e] = total;
        }
    }
    if (!arrives_last(&arrivals[blockIdx.x], (int)gridDim.y, &is_last)) return;
    for (int t = warp; t < count; t += ROUTER_WARPS) {
        const size_t token = (size_t)(first + t);
        choose_experts(gates + token * experts, logits_s + warp * ROUTER_SCRATCH(experts), chosen_ids ? chosen_ids + token * top : nullptr,
                       chosen_weights ? chosen_weights + token * top : nullptr, experts, top, lane, rule);
    }
}

// Whether a rule fits the experts it is to choose among.
static bool router_rule_fits(const RouterRule& rule, int experts, int top) {
    if (rule.mode < 0 || rule.mode > 2) return false;
    if (rule.mode != 2) return true;
    if (rule.groups <= 0 || rule.keep <= 0 || rule.keep > rule.groups || experts % rule.groups != 0) return false;
    return top <= rule.keep * (experts / rule.groups);
}

template <typename T>
static int router_gates_launch(const void* x, long x_stride, const float* router, float* gates, int* chosen_ids,
                               float* chosen_weights, int* arrivals, int tokens, int hidden, int experts, int top,
                               RouterRule rule, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (experts <= 0 || top <= 0 || top > experts || hidden <= 0 || experts > 1024 || !arrivals) return KIRAI_ERR_BAD_SIZE;
    if (!router_rule_fits(rule, experts, top)) return KIRAI_ERR_BAD_SIZE;
    if ((chosen_ids == nullptr) != (chosen_weights == nullptr)) return KIRAI_ERR_BAD_SIZE;
    if (tokens * (long)experts <= 4096 && experts <= 65535) {
        return launch_pdl(router_gates_few_kernel<T>, dim3(tokens, experts), dim3(ROUTER_WARPS * 32), ROUTER_SCRATCH(experts) * sizeof(float),
                          stream, 1u, (const T*)x, x_stride, router, gates, chosen_ids, chosen_weights, arrivals, hidden, experts, top, rule);
    }
    const unsigned slices = (unsigned)((experts + ROUTER_WARPS - 1) / ROUTER_WARPS);
    const unsigned groups = (unsigned)((tokens + ROUTER_TOKENS - 1) / ROUTER_TOKENS);
    return launch_pdl(router_gates_many_kernel<T>, dim3(groups, slices), dim3(ROUTER_WARPS * 32),
                      ROUTER_WARPS * ROUTER_SCRATCH(experts) * sizeof(float), stream, 1u, (const T*)x, x_stride, router, gates, chosen_ids,
                      chosen_weights, arrivals, tokens, hidden, experts, top, rule);
}

// The choice alone, for logits that a product left in `gates` [tokens, experts]: a warp per token.
__global__ void __launch_bounds__(ROUTER_WARPS * 32)
router_choose_kernel(float* __restrict__ gates, int* __restrict__ chosen_ids, float* __restrict__ chosen_weights, int tokens,
                     int experts, int top, RouterRule rule) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float logits_s[];  // [ROUTER_WARPS][experts]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t token = (size_t)blockIdx.x * ROUTER_WARPS + warp;
    if (token >= (size_t)tokens) return;
    choose_experts(gates + token * experts, logits_s + warp * ROUTER_SCRATCH(experts), chosen_ids ? chosen_ids + token * top : nullptr,
                   chosen_weights ? chosen_weights + token * top : nullptr, experts, top, lane, rule);
}

// gates [tokens, experts] holds router logits (32-bit) and receives the routing weights; see router_gates.
// rule, correction, groups, keep: see RouterRule.
KIRAI_EXPORT int kirai_router_choose(float* gates, int* chosen_ids, float* chosen_weights, int tokens, int experts, int top,
                                     int rule, const float* correction, int groups, int keep, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (experts <= 0 || top <= 0 || top > experts || experts > 1024) return KIRAI_ERR_BAD_SIZE;
    if ((chosen_ids == nullptr) != (chosen_weights == nullptr)) return KIRAI_ERR_BAD_SIZE;
    const RouterRule how{rule, correction, groups, keep};
    if (!router_rule_fits(how, experts, top)) return KIRAI_ERR_BAD_SIZE;
    return launch_pdl(router_choose_kernel, dim3((unsigned)((tokens + ROUTER_WARPS - 1) / ROUTER_WARPS)), dim3(ROUTER_WARPS * 32),
                      ROUTER_WARPS * ROUTER_SCRATCH(experts) * sizeof(float), stream, 1u, gates, chosen_ids, chosen_weights, tokens, experts, top, how);
}

// arrivals [tokens]: zero before the first launch; every launch leaves it zero.
KIRAI_EXPORT int kirai_router_gates_f32(const void* x, long x_stride, const float* router, float* gates, int* chosen_ids,
                                        float* chosen_weights, int* arrivals, int tokens, int hidden, int experts, int top,
                                        int rule, const float* correction, int groups, int keep, cudaStream_t stream) {
    return router_gates_launch<float>(x, x_stride, router, gates, chosen_ids, chosen_weights, arrivals, tokens, hidden, experts, top,
                                      RouterRule{rule, correction, groups, keep}, stream);
}
KIRAI_EXPORT int kirai_router_gates_bf16(const void* x, long x_stride, const float* router, float* gates, int* chosen_ids,
                                         float* chosen_weights, int* arrivals, int tokens, int hidden, int experts, int top,
                                         int rule, const float* correction, int groups, int keep, cudaStream_t stream) {
    return router_gates_launch<bf16>(x, x_stride, router, gates, chosen_ids, chosen_weights, arrivals, tokens, hidden, experts, top,
                                     RouterRule{rule, correction, groups, keep}, stream);
}

// activation: 0 = relu(z)^2
template <typename T>
__global__ void expert_activation_gate_kernel(T* __restrict__ up, const float* __restrict__ gates, long rows, int experts, int ff) {
    pdl_launch_dependents();
    pdl_wait();
    const long width = (long)experts * ff;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * width) return;
    const long row = idx / width;
    const int expert = (int)((idx - row * width) / ff);
    const float gate = gates[row * experts + expert];
    float z = to_f32<T>(up[idx]);
    z = z > 0.0f ? z * z : 0.0f;
    up[idx] = from_f32<T>(gate == 0.0f ? 0.0f : z * gate);  // an expert that was not chosen gives zeros whatever it computed
}

template <typename T>
static int expert_activation_gate_launch(void* up, const float* gates, int rows, int experts, int ff, cudaStream_t stream) {
    const long total = (long)rows * experts * ff;
    if (total <= 0) return 0;
    return launch_pdl(expert_activation_gate_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, 1u, (T*)up,
                      gates, (long)rows, experts, ff);
}

// up [T, experts * ff] in place: relu(z)^2 times the token's gate of the column's expert.
KIRAI_EXPORT int kirai_relu2_gate_f32(void* up, const float* gates, int rows, int experts, int ff, cudaStream_t stream) {
    return expert_activation_gate_launch<float>(up, gates, rows, experts, ff, stream);
}
KIRAI_EXPORT int kirai_relu2_gate_bf16(void* up, const float* gates, int rows, int experts, int ff, cudaStream_t stream) {
    return expert_activation_gate_launch<bf16>(up, gates, rows, experts, ff, stream);
}

// ---------------------------------------------------------------------------------------------------------------
// Rows sorted by expert, for many tokens: every (token, chosen expert) pair gets a row ("slot") in a buffer whose
// experts' stretches are padded to whole tiles of 128 rows, so that a grouped product multiplies each tile with one
// expert's matrices and only the chosen experts' arithmetic is done.
//
//   route_plan     one block: counts the pairs of every expert, lays the experts' stretches one after the other (each a
//                  whole number of tiles), writes tile_group [max_tiles] (the expert of each tile; tiles behind the last
//                  stretch get -1 and hold no rows), slot_of [T, top] and row_of_slot [max_tiles * 128] (-1: padding).
//                  Which slot of its expert's stretch a pair gets depends on the order in which threads arrive; rows of a
//                  product are independent, so results do not.
//   route_gather   sorted[slot] = x[row_of_slot[slot]] (zeros for padding).
//   route_combine  out[t] = sum_j weight[t, j] * y[slot_of[t, j]] in 32-bit, in the order of choice.
#define PLAN_THREADS 1024
#define ROUTE_TILE 128

__global__ void __launch_bounds__(PLAN_THREADS)
route_plan_kernel(const int* __restrict__ chosen_ids, int* __restrict__ tile_group, int* __restrict__ slot_of,
                  int* __restrict__ row_of_slot, int tokens, int top, int experts, int max_tiles) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ int plan_s[];  // counts [experts], offsets [experts], cursors [experts]
    int* counts = plan_s;
    int* offsets = plan_s + experts;
    int* cursors = plan_s + 2 * experts;
    const int pairs = tokens * top;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = cursors[e] = 0;
    for (int i = threadIdx.x; i < max_tiles * ROUTE_TILE; i += blockDim.x) row_of_slot[i] = -1;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = chosen_ids[p];
        if (e >= 0 && e < experts) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int tile = 0;
        for (int e = 0; e < experts; ++e) {
            offsets[e] = tile * ROUTE_TILE;
            const int tiles = (counts[e] + ROUTE_TILE - 1) / ROUTE_TILE;
            for (int t = 0; t < tiles && tile < max_tiles; ++t) tile_group[tile++] = e;
        }
        for (; tile < max_tiles; ++tile) tile_group[tile] = -1;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = chosen_ids[p];
        int slot = -1;
        if (e >= 0 && e < experts) {
            slot = offsets[e] + atomicAdd(&cursors[e], 1);
            if (slot < max_tiles * ROUTE_TILE) row_of_slot[slot] = p / top;
            else slot = -1;
        }
        slot_of[p] = slot;
    }
}

KIRAI_EXPORT int kirai_route_plan(const int* chosen_ids, int* tile_group, int* slot_of, int* row_of_slot, int tokens, int top,
                                  int experts, int max_tiles, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (experts <= 0 || experts > 4096 || top <= 0 || max_tiles < (tokens * top + ROUTE_TILE - 1) / ROUTE_TILE + experts - 1)
        return KIRAI_ERR_BAD_SIZE;
    return launch_pdl(route_plan_kernel, dim3(1), dim3(PLAN_THREADS), (size_t)3 * experts * sizeof(int), stream, 1u, chosen_ids,
                      tile_group, slot_of, row_of_slot, tokens, top, experts, max_tiles);
}

__global__ void route_gather_kernel(const bf16* __restrict__ x, long x_stride, const int* __restrict__ row_of_slot,
                                    bf16* __restrict__ sorted, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    const int slot = blockIdx.x;
    const int row = row_of_slot[slot];
    bf16* dst = sorted + (size_t)slot * hidden;
    const bf16* src = x + (size_t)(row < 0 ? 0 : row) * x_stride;
    if (hidden % 8 == 0 && x_stride % 8 == 0 && (((uintptr_t)x | (uintptr_t)sorted) & 15) == 0) {
        for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x)
            reinterpret_cast<uint4*>(dst)[i] = row < 0 ? make_uint4(0u, 0u, 0u, 0u) : reinterpret_cast<const uint4*>(src)[i];
        return;
    }
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = row < 0 ? __float2bfloat16_rn(0.0f) : src[i];
}

KIRAI_EXPORT int kirai_route_gather_bf16(const void* x, long x_stride, const int* row_of_slot, void* sorted, int slots, int hidden,
                                         cudaStream_t stream) {
    if (slots <= 0 || hidden <= 0) return 0;
    return launch_pdl(route_gather_kernel, dim3(slots), dim3(hidden >= 2048 ? 256 : 128), 0, stream, 1u, (const bf16*)x, x_stride,
                      row_of_slot, (bf16*)sorted, hidden);
}

template <typename T>
__global__ void route_combine_kernel(const T* __restrict__ y, const int* __restrict__ slot_of, const float* __restrict__ weights,
                                     float* __restrict__ out, int hidden, int top) {
    pdl_launch_dependents();
    pdl_wait();
    const int token = blockIdx.x;
    if (hidden % 4 == 0 && (((uintptr_t)y | (uintptr_t)out) & 15) == 0) {
        for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (int j = 0; j < top; ++j) {
                const int slot = slot_of[(size_t)token * top + j];
                if (slot < 0) continue;
                const float w = weights[(size_t)token * top + j];
                const float4 v = load4(y + (size_t)slot * hidden + i);
                acc.x = fmaf(w, v.x, acc.x), acc.y = fmaf(w, v.y, acc.y), acc.z = fmaf(w, v.z, acc.z), acc.w = fmaf(w, v.w, acc.w);
            }
            *reinterpret_cast<float4*>(out + (size_t)token * hidden + i) = acc;
        }
        return;
    }
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float acc = 0.0f;
        for (int j = 0; j < top; ++j) {
            const int slot = slot_of[(size_t)token * top + j];
            if (slot >= 0) acc = fmaf(weights[(size_t)token * top + j], to_f32<T>(y[(size_t)slot * hidden + i]), acc);
        }
        out[(size_t)token * hidden + i] = acc;
    }
}

KIRAI_EXPORT int kirai_route_combine_bf16(const void* y, const int* slot_of, const float* weights, float* out, int tokens,
                                          int hidden, int top, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    return launch_pdl(route_combine_kernel<bf16>, dim3(tokens), dim3(hidden >= 2048 ? 256 : 128), 0, stream, 1u, (const bf16*)y,
                      slot_of, weights, out, hidden, top);
}
KIRAI_EXPORT int kirai_route_combine_f32(const void* y, const int* slot_of, const float* weights, float* out, int tokens,
                                         int hidden, int top, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    return launch_pdl(route_combine_kernel<float>, dim3(tokens), dim3(hidden >= 2048 ? 256 : 128), 0, stream, 1u, (const float*)y,
                      slot_of, weights, out, hidden, top);
}

// route_combine and the norm on the feed-forward's output in one pass: row t of the experts' result is
// sum_j weight[t, j] * y[slot_of[t, j]] in 32-bit (never written out), and stream[t] += row * rsqrt(mean(row^2) + eps) *
// norm_weight; copy[t] = bf16(stream[t]).  One block per token, the row in registers (width a multiple of 4, at most
// 4 * VEC * blockDim values).
template <int VEC>
__global__ void route_combine_norm_add_kernel(float* __restrict__ resid, const bf16* __restrict__ y, const int* __restrict__ slot_of,
                                              const float* __restrict__ weights, const float* __restrict__ norm_weight,
                                              bf16* __restrict__ copy, int hidden, int top, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const int token = blockIdx.x;
    const int quads = hidden >> 2;
    float4 kept[VEC];
    float acc = 0.0f;
#pragma unroll
    for (int n = 0; n < VEC; ++n) {
        const int i = threadIdx.x + n * blockDim.x;
        kept[n] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (i < quads) {
            for (int j = 0; j < top; ++j) {
                const int slot = slot_of[(size_t)token * top + j];
                if (slot < 0) continue;
                const float w = weights[(size_t)token * top + j];
                const float4 v = load4(y + (size_t)slot * hidden + 4 * (size_t)i);
                kept[n].x = fmaf(w, v.x, kept[n].x), kept[n].y = fmaf(w, v.y, kept[n].y);
                kept[n].z = fmaf(w, v.z, kept[n].z), kept[n].w = fmaf(w, v.w, kept[n].w);
            }
            acc += (kept[n].x * kept[n].x + kept[n].y * kept[n].y) + (kept[n].z * kept[n].z + kept[n].w * kept[n].w);
        }
    }
    const float variance = block_sum(acc, scratch) / (float)hidden + eps;
    const float scale = variance == 0.0f ? 0.0f : 1.0f / sqrtf(variance);
    float4* dst = reinterpret_cast<float4*>(resid + (size_t)token * hidden);
    const float4* w4 = reinterpret_cast<const float4*>(norm_weight);
#pragma unroll
    for (int n = 0; n < VEC; ++n) {
        const int i = threadIdx.x + n * blockDim.x;
        if (i < quads) {
            float4 r = dst[i];
            const float4 w = w4[i];
            r.x += kept[n].x * scale * w.x, r.y += kept[n].y * scale * w.y, r.z += kept[n].z * scale * w.z, r.w += kept[n].w * scale * w.w;
            dst[i] = r;
            if (copy) {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(r.x, r.y), hi = __floats2bfloat162_rn(r.z, r.w);
                uint2 packed;
                packed.x = *reinterpret_cast<const uint32_t*>(&lo);
                packed.y = *reinterpret_cast<const uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(copy + (size_t)token * hidden + 4 * (size_t)i) = packed;
            }
        }
    }
}

// Refuses (KIRAI_ERR_UNSUPPORTED) widths that are no multiple of 4 or above 8,192 and buffers off 16-byte boundaries: the
// caller then runs route_combine and the norm kernel one after the other.
KIRAI_EXPORT int kirai_route_combine_norm_add_bf16(float* resid, const void* y, const int* slot_of, const float* weights,
                                                   const float* norm_weight, void* copy, int tokens, int hidden, int top, float eps,
                                                   cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (hidden <= 0 || top <= 0) return KIRAI_ERR_BAD_SIZE;
    if (hidden % 4 != 0 || hidden > 4 * 4 * 512 ||
        (((uintptr_t)resid | (uintptr_t)y | (uintptr_t)norm_weight | (uintptr_t)copy) & 15) != 0)
        return KIRAI_ERR_UNSUPPORTED;
    const int threads = hidden <= 4 * 4 * 128 ? 128 : (hidden <= 4 * 4 * 256 ? 256 : 512);
    return launch_pdl(route_combine_norm_add_kernel<4>, dim3(tokens), dim3(threads), 0, stream, 1u, resid, (const bf16*)y, slot_of,
                      weights, norm_weight, (bf16*)copy, hidden, top, eps);
}
