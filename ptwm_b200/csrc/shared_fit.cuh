// Shared Order1ScaleAC states for the scale planes of a model (the writer's
// passes 2 and 3: crates/ptwm-core/src/compressor.rs:834-939, fit/order1.rs).
//
// Every scale plane brings its lag-1 counts (from the device, o1sac_count_kernel).
// Pass 2 fits one state per plane, measures how far the planes' states are from
// one another (a symmetrised KL divergence over all 256 contexts, on the GPU:
// one block per pair of planes), merges the closest planes step by step
// (average linkage) and keeps the number of clusters, 1..8, whose pooled states
// describe all planes in the fewest bits, the states' own bytes included.
// Pass 3 then lets every scale plane choose between what it had and a payload
// coded against one of the shared states, whose bytes it does not have to carry.
#pragma once
#include <array>
#include <cmath>
#include <cstdint>
#include <string>
#include <vector>

#include "encode_tables.cuh"

namespace ptwm {

constexpr uint32_t FIT_TOTAL = 4096;  // quantize.rs ORDER1_QUANT_TOTAL
constexpr int FIT_K_MAX = 8;          // fit/order1.rs:9

struct FitCounts {                 // one scale plane
    const uint32_t* joint;         // [256][256]: joint[prev][cur]
    const uint32_t* marginal;      // [256]: first symbol of every row
};
struct FitState {                  // order1_scale_ac.rs StateV0
    uint8_t bitmap[32];
    uint16_t marginal[256];
    std::vector<std::array<uint16_t, 256>> rows;  // present contexts in increasing order
    const uint16_t* row_or_marginal(int prev) const {
        if (!((bitmap[prev >> 3] >> (prev & 7)) & 1)) return marginal;
        int r = 0;
        for (int b = 0; b < (prev >> 3); ++b) r += __builtin_popcount(bitmap[b]);
        r += __builtin_popcount(uint32_t(bitmap[prev >> 3]) & ((1u << (prev & 7)) - 1));
        return rows[size_t(r)].data();
    }
    std::vector<uint8_t> serialize() const {  // order1_scale_ac.rs:143-160: bitmap, marginal, rows, u16 little-endian
        std::vector<uint8_t> out(bitmap, bitmap + 32);
        auto put = [&](const uint16_t* p) { for (int i = 0; i < 256; ++i) { out.push_back(uint8_t(p[i])); out.push_back(uint8_t(p[i] >> 8)); } };
        put(marginal);
        for (auto& r : rows) put(r.data());
        return out;
    }
};

// order1_scale_ac.rs:997-1030: the marginal always, a row for every context seen at least once
inline FitState fit_quantize(const uint32_t* joint, const uint32_t* marginal) {
    FitState s{};
    quantize_pmf256(marginal, FIT_TOTAL, s.marginal);
    for (int prev = 0; prev < 256; ++prev) {
        uint64_t sum = 0;
        for (int i = 0; i < 256; ++i) sum += joint[256 * prev + i];
        if (uint32_t(sum) == 0) continue;  // the reference sums in u32
        s.bitmap[prev >> 3] |= uint8_t(1u << (prev & 7));
        s.rows.emplace_back();
        quantize_pmf256(joint + 256 * prev, FIT_TOTAL, s.rows.back().data());
    }
    return s;
}

// Bits the plane's symbols cost under `state` (fit/order1.rs:233-262): contexts in order, symbols in order, then the row starts.
inline double fit_cross_entropy_bits(const FitCounts& c, const FitState& state) {
    double bits = 0;
    for (int prev = 0; prev < 256; ++prev) {
        const uint32_t* jr = c.joint + 256 * prev;
        const uint16_t* row = nullptr;
        for (int cur = 0; cur < 256; ++cur) {
            const uint32_t n = jr[cur];
            if (!n) continue;
            if (!row) row = state.row_or_marginal(prev);
            const double prob = double(row[cur]) / double(FIT_TOTAL);
            if (prob > 0.0) bits += double(n) * -std::log2(prob);
        }
    }
    for (int cur = 0; cur < 256; ++cur) {
        const uint32_t n = c.marginal[cur];
        if (!n) continue;
        const double prob = double(state.marginal[cur]) / double(FIT_TOTAL);
        if (prob > 0.0) bits += double(n) * -std::log2(prob);
    }
    return bits;
}

// Symmetrised KL divergence between the states of two planes, weighted by the mean of their marginals (fit/order1.rs:79-101).
// dense[k] = 257 rows of 256 u16 for plane k: row 0 the marginal, row 1 + prev the row a symbol after `prev` is coded with
// (the marginal again where the context has no row).  One block per pair, thread `prev` sums its context in symbol order,
// thread 0 adds the 256 terms in context order, as the reference's loops do.
__global__ void __launch_bounds__(256) fit_pair_distance_kernel(const uint16_t* __restrict__ dense, const uint32_t* __restrict__ pairs, double* __restrict__ dist) {
    const uint32_t a = pairs[2 * blockIdx.x], b = pairs[2 * blockIdx.x + 1];
    const uint16_t* P = dense + size_t(a) * 257 * 256;
    const uint16_t* Q = dense + size_t(b) * 257 * 256;
    const uint32_t prev = threadIdx.x;
    const uint16_t* p = P + 256 * (1 + prev);
    const uint16_t* q = Q + 256 * (1 + prev);
    double kl_pq = 0, kl_qp = 0;
    for (int i = 0; i < 256; ++i) {
        const double pp = double(p[i]) / 4096.0, qq = double(q[i]) / 4096.0;
        if (pp > 0.0 && qq > 0.0) { kl_pq += pp * log(pp / qq); kl_qp += qq * log(qq / pp); }
    }
    const double ln2 = 0.693147180559945309417232121458;
    const double mix = 0.5 * (double(P[prev]) / 4096.0 + double(Q[prev]) / 4096.0);
    __shared__ double term[256];
    term[prev] = mix * (kl_pq / ln2 + kl_qp / ln2);
    __syncthreads();
    if (prev == 0) {
        double total = 0;
        for (int i = 0; i < 256; ++i) total += term[i];
        dist[blockIdx.x] = total;
    }
}

struct FitMerge { size_t left, right; };
// Average-linkage agglomeration over a full distance matrix (fit/order1.rs:126-176): the closest active pair, first in (i, j) order.
inline std::vector<FitMerge> fit_agglomerate(std::vector<double> dist, size_t n) {
    std::vector<FitMerge> merges;
    if (n < 2) return merges;
    std::vector<size_t> sizes(n, 1);
    std::vector<char> active(n, 1);
    for (size_t step = 0; step + 1 < n; ++step) {
        size_t bl = 0, br = 1;
        double best = INFINITY;
        for (size_t i = 0; i < n; ++i) {
            if (!active[i]) continue;
            for (size_t j = i + 1; j < n; ++j) {
                if (!active[j]) continue;
                if (dist[i * n + j] < best) { best = dist[i * n + j]; bl = i; br = j; }
            }
        }
        merges.push_back({bl, br});
        const double sl = double(sizes[bl]), sr = double(sizes[br]);
        for (size_t k = 0; k < n; ++k) {
            if (k == bl || k == br || !active[k]) continue;
            const double d = (sl * dist[bl * n + k] + sr * dist[br * n + k]) / (sl + sr);
            dist[bl * n + k] = d; dist[k * n + bl] = d;
        }
        sizes[bl] += sizes[br];
        active[br] = 0;
    }
    return merges;
}
// Cluster number of every plane after the first n - k merges, clusters numbered by their smallest member (fit/order1.rs:178-213).
inline std::vector<uint16_t> fit_slice(const std::vector<FitMerge>& merges, size_t n, size_t k) {
    std::vector<size_t> parent(n);
    for (size_t i = 0; i < n; ++i) parent[i] = i;
    auto find = [&](size_t x) { while (parent[x] != x) x = parent[x]; return x; };
    const size_t n_merges = std::min(n - std::min(n, k), merges.size());
    for (size_t m = 0; m < n_merges; ++m) {
        const size_t rl = find(merges[m].left), rr = find(merges[m].right);
        if (rl != rr) parent[std::max(rl, rr)] = std::min(rl, rr);
    }
    std::vector<size_t> roots(n), unique;
    for (size_t i = 0; i < n; ++i) roots[i] = find(i);
    unique = roots;
    std::sort(unique.begin(), unique.end());
    unique.erase(std::unique(unique.begin(), unique.end()), unique.end());
    std::vector<uint16_t> assignment(n);
    for (size_t i = 0; i < n; ++i) assignment[i] = uint16_t(std::lower_bound(unique.begin(), unique.end(), roots[i]) - unique.begin());
    return assignment;
}

struct FitResult {
    std::vector<FitState> states;      // the shared states, in cluster order
    std::vector<std::string> names;    // "order1_scale_ac/cluster_i_of_k"
};
// `distances(pairs)` returns the divergence of every listed pair of planes' states (the GPU kernel above, or a host loop in a test).
template <class Distances>
inline FitResult fit_shared_order1(const std::vector<FitCounts>& planes, Distances&& distances) {
    FitResult out;
    const size_t n = planes.size();
    if (!n) return out;
    if (n == 1) {  // fit/order1.rs:324-337
        out.states.push_back(fit_quantize(planes[0].joint, planes[0].marginal));
        out.names.push_back("order1_scale_ac/cluster_0_of_1");
        return out;
    }
    std::vector<FitState> own;
    for (auto& p : planes) own.push_back(fit_quantize(p.joint, p.marginal));
    std::vector<uint32_t> pairs;
    for (size_t i = 0; i < n; ++i) for (size_t j = i + 1; j < n; ++j) { pairs.push_back(uint32_t(i)); pairs.push_back(uint32_t(j)); }
    const std::vector<double> d = distances(own, pairs);
    std::vector<double> dist(n * n, 0.0);
    for (size_t k = 0; k < d.size(); ++k) { dist[size_t(pairs[2 * k]) * n + pairs[2 * k + 1]] = d[k]; dist[size_t(pairs[2 * k + 1]) * n + pairs[2 * k]] = d[k]; }
    const std::vector<FitMerge> merges = fit_agglomerate(dist, n);
    double best_bits = 0;
    bool have = false;
    std::vector<uint32_t> pooled_joint, pooled_marg;
    for (size_t k = 1; k <= std::min<size_t>(FIT_K_MAX, n); ++k) {  // fit/order1.rs:343-357: fewest bits, the smaller k on ties
        const std::vector<uint16_t> assignment = fit_slice(merges, n, k);
        pooled_joint.assign(k * 65536, 0); pooled_marg.assign(k * 256, 0);
        for (size_t i = 0; i < n; ++i) {
            uint32_t* j = pooled_joint.data() + size_t(assignment[i]) * 65536;
            uint32_t* m = pooled_marg.data() + size_t(assignment[i]) * 256;
            for (int e = 0; e < 65536; ++e) j[e] += planes[i].joint[e];
            for (int e = 0; e < 256; ++e) m[e] += planes[i].marginal[e];
        }
        std::vector<FitState> states;
        double bits = 0;
        for (size_t c = 0; c < k; ++c) {
            states.push_back(fit_quantize(pooled_joint.data() + c * 65536, pooled_marg.data() + c * 256));
            bits += 8.0 * double(32 + 512 + 512 * states.back().rows.size());
        }
        for (size_t i = 0; i < n; ++i) bits += fit_cross_entropy_bits(planes[i], states[assignment[i]]);
        if (!std::isfinite(bits)) continue;
        if (!have || bits < best_bits) {
            have = true; best_bits = bits;
            out.states = std::move(states);
            out.names.clear();
            for (size_t c = 0; c < k; ++c) out.names.push_back("order1_scale_ac/cluster_" + std::to_string(c) + "_of_" + std::to_string(k));
        }
    }
    return out;
}

// The dense row table of a state for fit_pair_distance_kernel.
inline void fit_dense_rows(const FitState& s, uint16_t* out /* 257 * 256 */) {
    for (int i = 0; i < 256; ++i) out[i] = s.marginal[i];
    for (int prev = 0; prev < 256; ++prev) {
        const uint16_t* r = s.row_or_marginal(prev);
        for (int i = 0; i < 256; ++i) out[256 * (1 + prev) + i] = r[i];
    }
}

}  // namespace ptwm
