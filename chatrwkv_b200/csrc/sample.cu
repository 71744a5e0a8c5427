// Token sampling on the device, with the semantics of PIPELINE.sample_logits and of the penalty bookkeeping in
// PIPELINE.generate (rwkv_pip_package/src/rwkv/utils.py:55-135): ban list, presence / frequency penalties with
// decay, softmax, nucleus (top-p) cutoff, top-k, temperature, one draw.  The reference sorts the whole vocabulary
// on the host or with torch.argsort every token; here the token never leaves the GPU, so the sampler can sit in the
// CUDA graph of a decode step and feed the next step's embedding row.
//
// One cluster of 8 CTAs x 512 threads; thread g owns the contiguous ids [g*c, (g+1)*c), c = ceil(V / 4096) <= 16,
// in registers.  Nothing is sorted: the nucleus cutoff is the largest probability v with
// sum{p_i : p_i >= v} >= top_p, which is what `sorted_probs[argmax(cumsum >= top_p)]` picks (utils.py:66-67,
// 80-82), found by a search over the bit pattern of v, four bits (fifteen thresholds) per round; the k-th largest
// probability for top-k comes from the same search with counts instead of sums.  A round costs one cluster
// barrier: every CTA pushes its fifteen partial sums into every CTA's shared memory (remote stores), and every
// CTA adds the eight partials in rank order, so all CTAs take the same decisions.  Sums are taken in a fixed
// order: the same inputs give the same token.
//
// Differences from the reference that cannot be avoided: its cumulative sum runs in sorted order and ours in id
// order, so a cutoff that hinges on the last ulp of a sum may fall one value higher or lower; ties at the top-k
// boundary are kept by lowest id (the reference keeps whichever its sort put last); the draw is an inverse-CDF
// walk in id order on a uniform number supplied by the caller, not torch.multinomial's or numpy's stream.
// One quirk is kept: when no prefix of the sorted probabilities reaches top_p (top_p above the rounded total),
// `argmax` of an all-false array is 0 and the reference keeps only the most likely token; so do we.
#include "common.cuh"

namespace {

constexpr int kSampleCtas = 8;
constexpr int kSampleThreads = 512;
constexpr int kSampleWarps = kSampleThreads / 32;
constexpr int kSamplePer = 16;                       // ids per thread at most
constexpr int kSampleMaxV = kSampleCtas * kSampleThreads * kSamplePer;      // 65536
constexpr int kFan = 15;                             // thresholds per search round (four bits)

struct SampleArgs {
    int V;
    const float* logits;
    float temperature, top_p;
    int top_k;
    float* occurrence;             // [V] decayed occurrence weights, or NULL (no penalties)
    unsigned char* seen;           // [V] 1 once a token has been generated
    const unsigned char* banned;   // [V] or NULL
    const float* token_weight;     // [V] what a generated token adds to its occurrence (utils.py:115-122), NULL = 1
    float alpha_presence, alpha_frequency, alpha_decay;
    const float* uniforms;         // [n_uniforms] numbers in [0, 1)
    int n_uniforms;
    unsigned* counter;             // draws so far (device word); this call uses uniforms[counter % n_uniforms]
    long long* token_out;
    float* probs_out;              // [V] or NULL: the distribution the draw was made from, normalised
};

__device__ __forceinline__ uint32_t sm_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void push_f32(const float* local, unsigned cta, float v) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(sm_u32(local)), "r"(cta));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(r), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Shared state of one CTA.  `slot` receives every rank's partials ([parity][rank][value]); the parity lets a CTA
// start the next round's pushes while a slower one still reads this round's.
struct SampleShared {
    float warp_part[kSampleWarps][kFan + 1];
    float slot[2][kSampleCtas][kFan + 1];
    float prefix[kSampleWarps];
    int pick;
};

// Cluster-wide sums of NV values per thread (NV <= 16): every thread of every CTA gets the same totals.
template <int NV>
__device__ __forceinline__ void cluster_sum(SampleShared& sh, unsigned rank, int& parity, const float (&v)[NV], float (&out)[NV]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float w[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) w[i] = warp_sum(v[i]);
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < NV; ++i) sh.warp_part[warp][i] = w[i];
    }
    __syncthreads();
    if (threadIdx.x < NV * kSampleCtas) {            // thread (value i, destination CTA d): this CTA's partial, pushed to d
        const int i = threadIdx.x % NV, d = threadIdx.x / NV;
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < kSampleWarps; ++q) s += sh.warp_part[q][i];
        push_f32(&sh.slot[parity][rank][i], unsigned(d), s);
    }
    cluster_barrier();
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < kSampleCtas; ++q) s += sh.slot[parity][q][i];
        out[i] = s;
    }
    parity ^= 1;
}

__device__ __forceinline__ float cluster_max(SampleShared& sh, unsigned rank, int& parity, float v) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    if (lane == 0) sh.warp_part[warp][0] = v;
    __syncthreads();
    if (threadIdx.x < kSampleCtas) {
        float s = sh.warp_part[0][0];
#pragma unroll
        for (int q = 1; q < kSampleWarps; ++q) s = fmaxf(s, sh.warp_part[q][0]);
        push_f32(&sh.slot[parity][rank][0], threadIdx.x, s);
    }
    cluster_barrier();
    float s = sh.slot[parity][0][0];
#pragma unroll
    for (int q = 1; q < kSampleCtas; ++q) s = fmaxf(s, sh.slot[parity][q][0]);
    parity ^= 1;
    return s;
}

// Largest bit pattern v (as a non-negative float) with  sum{ w_i : p_i >= v } >= target,  w_i = p_i (COUNT = false)
// or 1 (COUNT = true); 0 if even v = 0 fails.  Eight rounds of four bits.
template <bool COUNT>
__device__ __forceinline__ float search_threshold(SampleShared& sh, unsigned rank, int& parity, const float (&p)[kSamplePer],
                                                  const bool (&valid)[kSamplePer], float target) {
    uint32_t v = 0;
#pragma unroll 1
    for (int shift = 28; shift >= 0; shift -= 4) {
        float part[kFan], tot[kFan];
#pragma unroll
        for (int j = 0; j < kFan; ++j) part[j] = 0.f;
#pragma unroll
        for (int i = 0; i < kSamplePer; ++i) {
            if (valid[i]) {
                const uint32_t bits = __float_as_uint(p[i]);
                const float w = COUNT ? 1.0f : p[i];
#pragma unroll
                for (int j = 0; j < kFan; ++j)
                    if (bits >= (v | (uint32_t(j + 1) << shift))) part[j] += w;
            }
        }
        cluster_sum<kFan>(sh, rank, parity, part, tot);
        int best = 0;
#pragma unroll
        for (int j = 0; j < kFan; ++j)
            if (tot[j] >= target) best = j + 1;         // the sums fall as j rises: the last that holds
        if (shift == 28 && best > 7) best = 7;          // bit 31 is the sign
        v |= uint32_t(best) << shift;
    }
    return __uint_as_float(v);
}

__global__ void __cluster_dims__(kSampleCtas, 1, 1) __launch_bounds__(kSampleThreads, 1) sample_kernel(const SampleArgs a) {
    __shared__ SampleShared sh;
    unsigned rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    int parity = 0;
    const int g = int(rank) * kSampleThreads + threadIdx.x;
    const int c = (a.V + kSampleCtas * kSampleThreads - 1) / (kSampleCtas * kSampleThreads);
    const int id0 = g * c;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // logits with the ban list and the penalties of the tokens generated so far (utils.py:97-100)
    float p[kSamplePer];
    bool valid[kSamplePer];
    float lmax = -INFINITY;
#pragma unroll
    for (int i = 0; i < kSamplePer; ++i) {
        const int id = id0 + i;
        valid[i] = i < c && id < a.V;
        p[i] = -INFINITY;
        if (valid[i]) {
            float l = a.logits[id];
            if (a.banned != nullptr && a.banned[id]) l = -INFINITY;
            if (a.occurrence != nullptr && a.seen[id]) l -= a.alpha_presence + a.occurrence[id] * a.alpha_frequency;
            p[i] = l;
            lmax = fmaxf(lmax, l);
        }
    }
    lmax = cluster_max(sh, rank, parity, lmax);

    // softmax in fp32 (utils.py:59)
    float one[1] = {0.f}, tot1[1];
#pragma unroll
    for (int i = 0; i < kSamplePer; ++i) {
        p[i] = valid[i] ? expf(p[i] - lmax) : 0.f;
        one[0] += p[i];
    }
    cluster_sum<1>(sh, rank, parity, one, tot1);
    const float inv_z = 1.0f / tot1[0];
    float pmax = 0.f;
    one[0] = 0.f;
#pragma unroll
    for (int i = 0; i < kSamplePer; ++i) {
        p[i] *= inv_z;
        one[0] += p[i];
        pmax = fmaxf(pmax, p[i]);
    }
    cluster_sum<1>(sh, rank, parity, one, tot1);
    const float total = tot1[0];
    pmax = cluster_max(sh, rank, parity, pmax);

    // temperature 0 means greedy: temperature 1, top_p 0 (utils.py:56-58)
    float temperature = a.temperature, top_p = a.top_p;
    if (temperature == 0.f) { temperature = 1.f; top_p = 0.f; }

    // nucleus cutoff (utils.py:64-68): probabilities below it are dropped
    float cutoff;
    if (top_p <= 0.f || !(total >= top_p)) cutoff = pmax;
    else cutoff = search_threshold<false>(sh, rank, parity, p, valid, top_p);

    // top-k (utils.py:69-70): everything but the k most likely is dropped; ties at the boundary by lowest id
    float kth = 0.f;
    int ties_kept = 0x7fffffff;
    const bool use_k = a.top_k > 0 && a.top_k < a.V;
    if (use_k) {
        kth = search_threshold<true>(sh, rank, parity, p, valid, float(a.top_k));
        float gt[1] = {0.f}, gtt[1];
#pragma unroll
        for (int i = 0; i < kSamplePer; ++i) gt[0] += (valid[i] && p[i] > kth) ? 1.f : 0.f;
        cluster_sum<1>(sh, rank, parity, gt, gtt);
        ties_kept = a.top_k - int(gtt[0]);
    }

    // Exclusive prefix over threads in id order, cluster-wide, of one value per thread.
    auto exclusive_prefix = [&](float mine, float& grand) {
        float incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += n;
        }
        if (lane == 31) sh.warp_part[warp][0] = incl;
        __syncthreads();
        if (threadIdx.x == 0) {
            float run = 0.f;
            for (int q = 0; q < kSampleWarps; ++q) { sh.prefix[q] = run; run += sh.warp_part[q][0]; }
            for (int d = 0; d < kSampleCtas; ++d) push_f32(&sh.slot[parity][rank][0], unsigned(d), run);
        }
        cluster_barrier();
        float before = 0.f, all = 0.f;
#pragma unroll
        for (int q = 0; q < kSampleCtas; ++q) {
            const float t = sh.slot[parity][q][0];
            if (q < int(rank)) before += t;
            all += t;
        }
        parity ^= 1;
        grand = all;
        return before + sh.prefix[warp] + (incl - mine);
    };

    bool keep[kSamplePer];
    {
        float my_ties = 0.f, dummy;
#pragma unroll
        for (int i = 0; i < kSamplePer; ++i) my_ties += (use_k && valid[i] && p[i] == kth) ? 1.f : 0.f;
        float tie_rank = use_k ? exclusive_prefix(my_ties, dummy) : 0.f;
#pragma unroll
        for (int i = 0; i < kSamplePer; ++i) {
            bool k = valid[i] && !(p[i] < cutoff);
            if (use_k && k) {
                if (p[i] < kth) k = false;
                else if (p[i] == kth) { k = tie_rank < float(ties_kept); tie_rank += 1.f; }
            }
            keep[i] = k;
        }
    }

    // temperature (utils.py:71-72), then one draw by inverse CDF in id order
    const float inv_t = 1.0f / temperature;
    float mine = 0.f;
#pragma unroll
    for (int i = 0; i < kSamplePer; ++i) {
        p[i] = keep[i] ? (temperature != 1.f ? powf(p[i], inv_t) : p[i]) : 0.f;
        mine += p[i];
    }
    float grand;
    const float before = exclusive_prefix(mine, grand);
    const unsigned draw = a.counter != nullptr ? *a.counter : 0u;
    const float u = (a.uniforms != nullptr && a.n_uniforms > 0) ? a.uniforms[draw % unsigned(a.n_uniforms)] : 0.5f;
    const float target = u * grand;
    if (a.probs_out != nullptr) {
        const float inv = grand > 0.f ? 1.0f / grand : 0.f;
#pragma unroll
        for (int i = 0; i < kSamplePer; ++i)
            if (valid[i]) a.probs_out[id0 + i] = p[i] * inv;
    }
    // the owner of the draw: the last thread (in id order) that has mass and starts at or below the target
    if (threadIdx.x == 0) sh.pick = -1;
    __syncthreads();
    if (mine > 0.f && before <= target) atomicMax(&sh.pick, int(threadIdx.x));
    __syncthreads();
    {
        // which CTA: the highest rank that found an owner; every CTA learns all ranks' answers through the slots
        if (threadIdx.x < kSampleCtas) push_f32(&sh.slot[parity][rank][0], threadIdx.x, float(sh.pick));
        cluster_barrier();
        int owner_rank = -1;
#pragma unroll
        for (int q = 0; q < kSampleCtas; ++q)
            if (sh.slot[parity][q][0] >= 0.f) owner_rank = q;
        parity ^= 1;
        if (owner_rank < 0) owner_rank = 0;              // no mass at all (every logit -inf): id 0
        if (int(rank) == owner_rank && int(threadIdx.x) == max(sh.pick, 0)) {
            float run = before;
            int chosen = -1, last = -1;
#pragma unroll
            for (int i = 0; i < kSamplePer; ++i) {
                if (p[i] > 0.f) {
                    last = id0 + i;
                    run += p[i];
                    if (chosen < 0 && target < run) chosen = id0 + i;
                }
            }
            if (chosen < 0) chosen = last >= 0 ? last : 0;
            *a.token_out = chosen;
            if (a.counter != nullptr) *a.counter = draw + 1u;
            if (a.occurrence != nullptr)                 // told to every CTA for the bookkeeping below (ids < 2^24: exact)
                for (int d = 0; d < kSampleCtas; ++d) push_f32(&sh.slot[parity][0][1], unsigned(d), float(chosen));
        }
    }
    // occurrence bookkeeping for the next call (utils.py:111-122): everything seen decays, then the new token is
    // added; each id is touched by the thread that owns it
    if (a.occurrence != nullptr) {
        cluster_barrier();
        const int tok = int(sh.slot[parity][0][1]);
#pragma unroll
        for (int i = 0; i < kSamplePer; ++i) {
            const int id = id0 + i;
            if (valid[i]) {
                const bool was = a.seen[id] != 0;
                float o = was ? a.occurrence[id] * a.alpha_decay : 0.f;
                if (id == tok) {
                    o += a.token_weight != nullptr ? a.token_weight[tok] : 1.0f;
                    a.seen[id] = 1;
                }
                if (was || id == tok) a.occurrence[id] = o;
            }
        }
    }
}

}  // namespace

extern "C" int rwkv_sample_logits(int64_t V, const float* logits, float temperature, float top_p, int64_t top_k,
                                  float* occurrence, unsigned char* seen, const unsigned char* banned, const float* token_weight,
                                  float alpha_presence, float alpha_frequency, float alpha_decay,
                                  const float* uniforms, int64_t n_uniforms, uint32_t* counter,
                                  int64_t* token_out, float* probs_out, void* stream) {
    RWKV_CHECK_ARG(V >= 1 && logits != nullptr && token_out != nullptr);
    RWKV_CHECK_ARG(temperature >= 0.f && top_k >= 0 && n_uniforms >= 0 && n_uniforms <= INT32_MAX);
    RWKV_CHECK_ARG((occurrence == nullptr) == (seen == nullptr));
    if (V > kSampleMaxV) return RWKV_ERR_UNSUPPORTED;
    SampleArgs a;
    a.V = int(V);
    a.logits = logits;
    a.temperature = temperature;
    a.top_p = top_p;
    a.top_k = top_k > V ? int(V) : int(top_k);
    a.occurrence = occurrence;
    a.seen = seen;
    a.banned = banned;
    a.token_weight = token_weight;
    a.alpha_presence = alpha_presence;
    a.alpha_frequency = alpha_frequency;
    a.alpha_decay = alpha_decay;
    a.uniforms = uniforms;
    a.n_uniforms = int(n_uniforms);
    a.counter = counter;
    a.token_out = reinterpret_cast<long long*>(token_out);
    a.probs_out = probs_out;
    sample_kernel<<<kSampleCtas, kSampleThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
    return rwkv_launch_status();
}
