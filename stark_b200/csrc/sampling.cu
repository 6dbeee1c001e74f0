// Stochastic sampling over one row of full-vocabulary logits, the device form of the reference's
// unified sampler (crates/stark-engine/src/backends/cpu/kernel/sampling/unified_sampling.rs:15-117):
// finite check -> temperature (with overflow centring) -> top-k / top-p / min-p as ONE prefix of the
// descending (value, then lower index) order -> Gumbel-max with Philox4x32-10 noise keyed by the seed
// (encodable_block/sampling/gumbel.rs:1-85) -> first index of the maximum.
//
// One CTA of 1024 threads.  Without filters everything is element-wise plus two block reductions.  With
// filters the row is sorted for real (stable LSD radix sort, 8-bit digits, warp-coalesced with
// match_any ranking), because the reference's cut depends on sequentially accumulated f32 sums in that
// order: exp(v - max) is evaluated in parallel, then one thread adds the terms in order (stopping once a
// term can no longer change the sum, which is exact for a descending sequence) and walks the prefix.
#include <algorithm>
#include <cmath>

#include "context.cuh"
#include "ops.cuh"

namespace sb {

namespace {

constexpr int kSampleThreads = 1024;
constexpr int kSampleWarps = kSampleThreads / 32;

__device__ inline void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
    c[0] = n0, c[1] = lo1, c[2] = n2, c[3] = lo0;
}

__device__ inline float gumbel_at(unsigned long long seed, uint32_t index, uint32_t vocab) {
    // revidx (gumbel.rs:66-80): the counter layout of a 1024-thread group drawing 4 words per counter
    const uint32_t thread_idx = index % 1024u, block_idx = index / 1024u;
    const uint32_t offset = ((vocab + 4095u) / 4096u) * thread_idx + block_idx / 4u, word = block_idx % 4u;
    uint32_t c[4] = {offset, 0u, 0u, 0u};
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    philox_round(c, k0, k1);
#pragma unroll
    for (int i = 0; i < 9; ++i) {
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
        philox_round(c, k0, k1);
    }
    const uint32_t w = max(c[word] >> 8, 1u);                  // unit_interval: 24 bits, never 0
    const float u = (float)w * (1.0f / 16777216.0f);
    return -logf(-logf(u));
}

// ascending radix order of this key = descending float order
__device__ inline uint32_t descending_key(float v) {
    const uint32_t u = __float_as_uint(v);
    const uint32_t asc = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ~asc;
}
__device__ inline float key_value(uint32_t key) {
    const uint32_t asc = ~key;
    return __uint_as_float((asc & 0x80000000u) ? (asc & 0x7fffffffu) : ~asc);
}

struct SampleParams {
    const void *logits;
    uint32_t io_type, vocab, flags, top_k;
    unsigned long long seed;
    float temperature, top_p, min_p;
    float *work;                 // [vocab]
    uint32_t *keys[2], *idx[2];  // [vocab] each (filters only)
    float *terms;                // [vocab] (filters only)
    uint32_t *out;
};

template <typename T, typename F>
__device__ inline T block_reduce(T v, F f, T *scratch /* [32] */) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = f(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if ((threadIdx.x & 31u) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    T r = scratch[0];
    for (int w = 1; w < kSampleWarps; ++w) r = f(r, scratch[w]);
    return r;
}

// Stable LSD radix sort of (key, id) pairs by key, ascending, 8-bit digits, by one CTA of kSampleThreads.
// The sorted pairs end in buffer 0.  counts: [256][kSampleWarps] shared words, uscratch: [32] shared words.
__device__ inline void sort_pairs(uint32_t *const (&keys)[2], uint32_t *const (&idx)[2], uint32_t V, uint32_t *counts,
                                  uint32_t *uscratch) {
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    // each warp owns a contiguous span, read 32 elements at a time: stable within the span by lane order
    const uint32_t span = (V + kSampleWarps - 1u) / kSampleWarps;
    const uint32_t lo = min(V, warp * span), hi = min(V, lo + span);
    for (uint32_t pass = 0; pass < 4; ++pass) {
        const uint32_t *kin = keys[pass & 1u], *iin = idx[pass & 1u];
        uint32_t *kout = keys[(pass & 1u) ^ 1u], *iout = idx[(pass & 1u) ^ 1u];
        const uint32_t shift = pass * 8u;
        for (uint32_t i = tid; i < 256u * kSampleWarps; i += kSampleThreads) counts[i] = 0;
        __syncthreads();
        for (uint32_t base = lo; base < hi; base += 32u) {
            const uint32_t i = base + lane;
            const bool live = i < hi;
            const uint32_t digit = live ? (kin[i] >> shift) & 255u : 256u + lane;  // idle lanes match nobody
            const uint32_t peers = __match_any_sync(0xffffffffu, digit);
            if (live && (peers & ((1u << lane) - 1u)) == 0) counts[digit * kSampleWarps + warp] += __popc(peers);
            __syncwarp();
        }
        __syncthreads();
        // exclusive scan over (digit major, warp minor): 8192 entries, 8 per thread
        uint32_t local[8], sum = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            local[j] = counts[tid * 8u + j];
            sum += local[j];
        }
        uint32_t incl = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= (uint32_t)o) incl += n;
        }
        if (lane == 31u) uscratch[warp] = incl;
        __syncthreads();
        uint32_t before = 0;
        for (uint32_t w = 0; w < warp; ++w) before += uscratch[w];
        uint32_t run = before + incl - sum;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            counts[tid * 8u + j] = run;
            run += local[j];
        }
        __syncthreads();
        for (uint32_t base = lo; base < hi; base += 32u) {
            const uint32_t i = base + lane;
            const bool live = i < hi;
            const uint32_t key = live ? kin[i] : 0u, id = live ? iin[i] : 0u;
            const uint32_t digit = live ? (key >> shift) & 255u : 256u + lane;
            const uint32_t peers = __match_any_sync(0xffffffffu, digit);
            const uint32_t rank = __popc(peers & ((1u << lane) - 1u));
            uint32_t start = 0;
            if (live) start = counts[digit * kSampleWarps + warp];
            __syncwarp();
            if (live) {
                kout[start + rank] = key;
                iout[start + rank] = id;
                if (rank == 0) counts[digit * kSampleWarps + warp] = start + __popc(peers);
            }
            __syncwarp();
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(kSampleThreads) unified_sampling_kernel(const SampleParams p) {
    extern __shared__ uint32_t counts[];  // [256][kSampleWarps] radix counters
    __shared__ float fscratch[32];
    __shared__ uint32_t uscratch[32];
    __shared__ uint32_t keep_count;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, V = p.vocab;
    const auto fmax2 = [](float a, float b) { return fmaxf(a, b); };

    // ---- load, finite check (unified_sampling.rs:42-45) ----
    int bad = 0;
    for (uint32_t i = tid; i < V; i += kSampleThreads) {
        const float v = p.io_type == STARK_B200_F32 ? reinterpret_cast<const float *>(p.logits)[i]
                                                     : bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(p.logits)[i]);
        p.work[i] = v;
        bad |= !isfinite(v);
    }
    if (__syncthreads_or(bad)) {
        if (tid == 0) *p.out = 0xffffffffu;
        return;
    }
    // ---- temperature (:59-77) ----
    if (p.flags & 2u) {
        const float recip = 1.0f / p.temperature;
        int over = 0;
        float mx = -INFINITY;
        for (uint32_t i = tid; i < V; i += kSampleThreads) {
            const float v = p.work[i];
            over |= !isfinite(v * recip);
            mx = fmaxf(mx, v);
        }
        const int center = __syncthreads_or(over);
        const float shift = center ? block_reduce(mx, fmax2, fscratch) : 0.0f;
        for (uint32_t i = tid; i < V; i += kSampleThreads) {
            float v = p.work[i];
            if (center) v -= shift;
            p.work[i] = v * recip;
        }
        __syncthreads();
    }
    // ---- filters (:79-99): sort, sequential sums, prefix ----
    if (p.flags & (4u | 8u | 16u)) {
        for (uint32_t i = tid; i < V; i += kSampleThreads) {
            const float v = p.work[i];
            p.keys[0][i] = descending_key(v == 0.0f ? 0.0f : v);  // -0 and +0 compare equal: one key for both
            p.idx[0][i] = i;
        }
        __syncthreads();
        sort_pairs(p.keys, p.idx, V, counts, uscratch);
        // four passes: the sorted pairs are back in buffer 0
        const uint32_t *skey = p.keys[0], *sidx = p.idx[0];
        const float top = key_value(skey[0]);
        for (uint32_t i = tid; i < V; i += kSampleThreads) {
            p.terms[i] = expf(key_value(skey[i]) - top);
            p.work[i] = -INFINITY;
        }
        __syncthreads();
        if (tid == 0) {
            float norm = 0.0f;
            for (uint32_t i = 0; i < V; ++i) {  // sequential f32 sum in sorted order (:84-85)
                const float next = norm + p.terms[i];
                if (next == norm && i > 0) break;  // descending terms: none of the rest can move the sum
                norm = next;
            }
            const float floor_value = (p.flags & 16u) ? top + logf(p.min_p) : -INFINITY;
            float mass = 0.0f;
            uint32_t n = 0;
            for (; n < V; ++n) {
                if (((p.flags & 4u) && n >= p.top_k) || ((p.flags & 8u) && mass >= p.top_p) ||
                    ((p.flags & 16u) && key_value(skey[n]) < floor_value))
                    break;
                mass += p.terms[n] / norm;
            }
            keep_count = n;
        }
        __syncthreads();
        for (uint32_t n = tid; n < keep_count; n += kSampleThreads) p.work[sidx[n]] = key_value(skey[n]);
        __syncthreads();
    }
    // ---- Gumbel-max (:101-106) and the first index of the maximum (:108-114) ----
    float best = -INFINITY;
    uint32_t bi = 0xffffffffu;
    for (uint32_t i = tid; i < V; i += kSampleThreads) {
        float v = p.work[i];
        if (p.flags & 1u) v += gumbel_at(p.seed, i, V);
        if (v > best || (v == best && i < bi) || bi == 0xffffffffu) {
            best = v;
            bi = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) {
            best = ov;
            bi = oi;
        }
    }
    __syncthreads();
    if (lane == 0) {
        fscratch[warp] = best;
        uscratch[warp] = bi;
    }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < kSampleWarps; ++w)
            if (fscratch[w] > best || (fscratch[w] == best && uscratch[w] < bi)) {
                best = fscratch[w];
                bi = uscratch[w];
            }
        *p.out = isfinite(best) ? bi : 0xffffffffu;
    }
}

// The generation worker's host sampler (crates/stark-generate/src/hybrid.rs:1122-1212) on the device:
// candidates = the first k of the descending total order (lower id first among equal bit patterns,
// :1265-1372), probabilities exp(f64((l - max) / temperature)) with the subtraction and division in f32
// (:138-165), the sequential f64 total, the min-p / top-p prefix (:1192-1204), one SplitMix64 draw scaled
// by the kept mass and a sequential scan (:1103-1111, :1134-1142).
//
// The partial sums S_n of the probabilities in candidate order serve the total, the prefix walk and the
// scan alike, and they are what fixes the result bit for bit, so one thread forms them in order.  Two
// things keep that short: once adding a term leaves S unchanged no later (smaller) term can change it, so
// every walk stops adding there; and the quotient S / total is only formed when S is within 1e-14 of the
// threshold, where the comparison could go either way.
__global__ void __launch_bounds__(kSampleThreads) ordered_sampling_kernel(const SampleParams p) {
    extern __shared__ uint32_t counts[];
    __shared__ uint32_t uscratch[32];
    __shared__ uint32_t first_below;
    const uint32_t tid = threadIdx.x, V = p.vocab;
    int bad = 0;
    for (uint32_t i = tid; i < V; i += kSampleThreads) {
        const float v = p.io_type == STARK_B200_F32 ? reinterpret_cast<const float *>(p.logits)[i]
                                                     : bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(p.logits)[i]);
        bad |= !isfinite(v);
        p.keys[0][i] = descending_key(v);  // signed zeros stay distinct, as under total_cmp
        p.idx[0][i] = i;
    }
    if (tid == 0) first_below = 0xffffffffu;
    if (__syncthreads_or(bad)) {
        if (tid == 0) *p.out = 0xffffffffu;
        return;
    }
    sort_pairs(p.keys, p.idx, V, counts, uscratch);
    const uint32_t *skey = p.keys[0], *sidx = p.idx[0];
    double *terms = reinterpret_cast<double *>(p.idx[1]);  // idx[1] and the f32 term array: 8 bytes per entry
    const uint32_t k = (p.flags & 4u) ? min(p.top_k, V) : V;
    const float top = key_value(skey[0]);
    const float temperature = (p.flags & 2u) ? p.temperature : 1.0f;
    const double min_p = (double)p.min_p;
    uint32_t below = 0xffffffffu;
    for (uint32_t i = tid; i < k; i += kSampleThreads) {
        const double t = exp((double)__fdiv_rn(__fsub_rn(key_value(skey[i]), top), temperature));
        terms[i] = t;
        if ((p.flags & 16u) && i > 0 && t < min_p) below = min(below, i);
    }
    if (below != 0xffffffffu) atomicMin(&first_below, below);
    __syncthreads();
    if (tid != 0) return;
    const uint32_t limit = min(k, first_below);  // the min-p cut: the first candidate after the top one below it
    // total; `live` = number of leading terms that still move the partial sums
    double total = 0.0;
    uint32_t live = k;
    for (uint32_t base = 0; base < k && live == k; base += 8u) {
        double t[8];
#pragma unroll
        for (uint32_t j = 0; j < 8u; ++j) t[j] = base + j < k ? terms[base + j] : 0.0;
#pragma unroll
        for (uint32_t j = 0; j < 8u; ++j) {
            if (base + j >= k) break;
            if (base + j > 0 && total + 2.0 * t[j] == total) {
                live = base + j;
                break;
            }
            total += t[j];
        }
    }
    // prefix: stop before candidate n > 0 once S_n / total >= top_p
    double cumulative = 0.0;
    uint32_t kept = 0;
    if (p.flags & 8u) {
        const double top_p = (double)p.top_p, edge = top_p * total;
        const double lo = edge * (1.0 - 1e-14), hi = edge * (1.0 + 1e-14);
        for (; kept < limit; ++kept) {
            if (kept > 0 && cumulative >= lo && (cumulative > hi || cumulative / total >= top_p)) break;
            if (kept >= live) {  // S no longer changes: neither does the comparison
                kept = limit;
                break;
            }
            cumulative += terms[kept];
        }
    } else {
        const uint32_t n = min(limit, live);
        for (uint32_t base = 0; base < n; base += 8u) {
            double t[8];
#pragma unroll
            for (uint32_t j = 0; j < 8u; ++j) t[j] = base + j < n ? terms[base + j] : 0.0;
#pragma unroll
            for (uint32_t j = 0; j < 8u; ++j)
                if (base + j < n) cumulative += t[j];
        }
        kept = limit;
    }
    // draw
    unsigned long long z = p.seed + 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    const double u = (double)((z ^ (z >> 31)) >> 11) * (1.0 / 9007199254740992.0);
    const double target = u * cumulative;
    uint32_t chosen = kept - 1u;
    double mass = 0.0;
    const uint32_t scan = min(kept, live);
    for (uint32_t n = 0; n < scan; ++n) {
        mass += terms[n];
        if (target < mass) {
            chosen = n;
            break;
        }
    }
    *p.out = sidx[chosen];
}

}  // namespace

size_t sampling_scratch_bytes(uint32_t vocab) { return (size_t)vocab * 4u * 6u; }

// SamplingMethod::validate (generation.rs:67-111): finite temperature in (0, 100] with a finite
// reciprocal, 1 <= top_k <= vocab, 0 < top_p <= 1, 0 <= min_p <= 1.
stark_b200_status sampling_validate(const stark_b200_sampling &s, uint32_t vocab) {
    if (vocab == 0 || (s.flags & ~63u)) return STARK_B200_INVALID_ARGUMENT;
    if ((s.flags & 32u) && !(s.flags & 1u)) return STARK_B200_INVALID_ARGUMENT;  // the ordered sampler only draws
    if (s.flags & 2u) {
        if (!std::isfinite(s.temperature) || !(s.temperature > 0.0f) || s.temperature > 100.0f ||
            !std::isfinite(1.0f / s.temperature))
            return STARK_B200_INVALID_ARGUMENT;
    }
    if ((s.flags & 4u) && (s.top_k < 1u || s.top_k > vocab)) return STARK_B200_INVALID_ARGUMENT;
    if ((s.flags & 8u) && !(s.top_p > 0.0f && s.top_p <= 1.0f)) return STARK_B200_INVALID_ARGUMENT;
    if ((s.flags & 16u) && !(s.min_p >= 0.0f && s.min_p <= 1.0f)) return STARK_B200_INVALID_ARGUMENT;
    return STARK_B200_OK;
}

stark_b200_status sampling_launch(const void *logits, uint32_t io_type, uint32_t vocab, const stark_b200_sampling &s,
                                  void *scratch, uint32_t *out_device, cudaStream_t stream) {
    stark_b200_status st = sampling_validate(s, vocab);
    if (st != STARK_B200_OK) return st;
    if (!logits || !scratch || !out_device || io_type > STARK_B200_F32) return STARK_B200_INVALID_ARGUMENT;
    SampleParams p{};
    p.logits = logits;
    p.io_type = io_type;
    p.vocab = vocab;
    p.flags = s.flags;
    p.top_k = s.top_k;
    p.seed = s.seed;
    p.temperature = s.temperature;
    p.top_p = s.top_p;
    p.min_p = s.min_p;
    uint32_t *base = static_cast<uint32_t *>(scratch);
    p.work = reinterpret_cast<float *>(base);
    p.keys[0] = base + vocab;
    p.keys[1] = base + 2u * (size_t)vocab;
    p.idx[0] = base + 3u * (size_t)vocab;
    p.idx[1] = base + 4u * (size_t)vocab;
    p.terms = reinterpret_cast<float *>(base + 5u * (size_t)vocab);
    p.out = out_device;
    const size_t smem = 256u * kSampleWarps * sizeof(uint32_t);
    if (s.flags & 32u)
        ordered_sampling_kernel<<<1, kSampleThreads, smem, stream>>>(p);
    else
        unified_sampling_kernel<<<1, kSampleThreads, smem, stream>>>(p);
    SB_CUDA(cudaGetLastError());
    return STARK_B200_OK;
}

}  // namespace sb
