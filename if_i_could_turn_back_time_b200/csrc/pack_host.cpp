// Host-side packers: fp32 weights -> packed E2M1 / GF4 (CPU, multi-threaded).
// One-off work at model load, not the inference hot path.
//
// GF4 codebooks come from an exact 16-class Jenks natural-breaks partition of
// each group-normalised row.  The partition minimises the within-class sum of
// squared deviations over contiguous classes of the ascending-sorted row (the
// objective the reference evaluates for two classes in
// Python_Jenks_Test/Jenks_Tests/cuda_helpers.py:151-184), here through the
// divide-and-conquer form of the dynamic programme: the left-most optimal
// split point is monotone in the prefix length, so each DP layer costs
// O(m log m) segment evaluations instead of O(m^2).
#include <algorithm>
#include <atomic>
#include <cfloat>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "../../include/jq.h"

namespace {

inline int stride_codes(int K) { return (K + 31) / 32 * 32; }

// IEEE double -> binary16 bits, round to nearest even, single rounding.
uint16_t double_to_half_bits(double d) {
    uint16_t sign = std::signbit(d) ? 0x8000u : 0u;
    double a = std::fabs(d);
    if (std::isnan(d)) return (uint16_t)(sign | 0x7e00u);
    if (a >= 65520.0) return (uint16_t)(sign | 0x7c00u);
    if (a < 6.103515625e-05) {  // below 2^-14: subnormal grid of 2^-24
        double m = std::nearbyint(std::ldexp(a, 24));
        return (uint16_t)(sign | (uint16_t)m);  // m == 1024 is the smallest normal
    }
    int e;
    (void)std::frexp(a, &e);  // a = f * 2^e, f in [0.5, 1)
    e -= 1;                   // a in [2^e, 2^(e+1))
    double m = std::nearbyint(std::ldexp(a, 10 - e));  // in [1024, 2048]
    if (m >= 2048.0) { m = 1024.0; e += 1; }
    if (e > 15) return (uint16_t)(sign | 0x7c00u);
    return (uint16_t)(sign | (uint16_t)((e + 15) << 10) | ((uint16_t)m - 1024u));
}

float half_bits_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const int exp = (h >> 10) & 0x1f;
    const uint32_t man = h & 0x3ffu;
    float out;
    if (exp == 0) {
        out = std::ldexp((float)man, -24);
    } else if (exp == 31) {
        out = man ? NAN : INFINITY;
    } else {
        out = std::ldexp((float)(man | 0x400u), exp - 25);
    }
    uint32_t bits;
    std::memcpy(&bits, &out, 4);
    bits |= sign;
    std::memcpy(&out, &bits, 4);
    return out;
}

// nearest E2M1 code, ties to the even mantissa bit, saturating; never code 8
inline uint8_t e2m1_code(float u) {
    const float a = std::fabs(u);
    int idx;
    if (a < 0.25f) idx = 0;
    else if (a == 0.25f) idx = 0;
    else if (a < 0.75f) idx = 1;
    else if (a == 0.75f) idx = 2;
    else if (a < 1.25f) idx = 2;
    else if (a == 1.25f) idx = 2;
    else if (a < 1.75f) idx = 3;
    else if (a == 1.75f) idx = 4;
    else if (a < 2.5f) idx = 4;
    else if (a == 2.5f) idx = 4;
    else if (a < 3.5f) idx = 5;
    else if (a == 3.5f) idx = 6;
    else if (a < 5.0f) idx = 6;
    else if (a == 5.0f) idx = 6;
    else idx = 7;  // includes NaN-free saturation above 6
    return (uint8_t)((u < 0 && idx != 0) ? idx + 8 : idx);
}

template <class F>
void parallel_rows(int N, int threads, F fn) {
    int T = threads > 0 ? threads : (int)std::thread::hardware_concurrency();
    if (T < 1) T = 1;
    if (T > N) T = N;
    std::atomic<int> next(0);
    auto work = [&]() {
        for (;;) {
            int n = next.fetch_add(1);
            if (n >= N) break;
            fn(n);
        }
    };
    if (T == 1) { work(); return; }
    std::vector<std::thread> pool;
    pool.reserve(T);
    for (int t = 0; t < T; ++t) pool.emplace_back(work);
    for (auto &th : pool) th.join();
}

inline void put_code(uint8_t *rowbytes, int k, uint8_t c) {
    // rows are zeroed first; codes may arrive in any order
    rowbytes[k >> 1] = (uint8_t)(rowbytes[k >> 1] | ((k & 1) ? (c << 4) : c));
}

// ---- Jenks k-class on (distinct value, multiplicity) pairs ------------------
struct Jenks {
    std::vector<double> P1, P2, C, prev, cur;
    std::vector<int> arg;  // (k+1) x (m+1)
    int m = 0;

    inline double cost(int a, int b) const {
        const double d1 = P1[b] - P1[a];
        const double d2 = P2[b] - P2[a];
        const double c = C[b] - C[a];
        const double sq = d1 * d1;
        const double q = sq / c;
        return d2 - q;
    }

    // fill cur[i], arg[j][i] for i in [lo, hi] knowing the split lies in [optlo, opthi]
    void solve(int j, int lo, int hi, int optlo, int opthi) {
        // explicit stack: recursion depth is only log2(m), but this keeps frames tiny
        struct Fr { int lo, hi, optlo, opthi; };
        std::vector<Fr> st;
        st.push_back({lo, hi, optlo, opthi});
        while (!st.empty()) {
            Fr f = st.back();
            st.pop_back();
            if (f.lo > f.hi) continue;
            const int mid = (f.lo + f.hi) >> 1;
            const int t0 = std::max(f.optlo, j - 1), t1 = std::min(mid - 1, f.opthi);
            double best = DBL_MAX;
            int bt = t0;
            for (int t = t0; t <= t1; ++t) {
                const double c = prev[t] + cost(t, mid);
                if (c < best) { best = c; bt = t; }
            }
            cur[mid] = best;
            arg[(size_t)j * (m + 1) + mid] = bt;
            st.push_back({f.lo, mid - 1, f.optlo, bt});
            st.push_back({mid + 1, f.hi, bt, f.opthi});
        }
    }

    // v ascending distinct, cnt multiplicities; returns classes used, fills breaks[0..ke]
    int run(const double *v, const double *cnt, int m_, int k, int *breaks) {
        m = m_;
        const int ke = std::min(k, m);
        P1.assign(m + 1, 0.0); P2.assign(m + 1, 0.0); C.assign(m + 1, 0.0);
        for (int t = 0; t < m; ++t) {
            const double cv = cnt[t] * v[t];
            const double cvv = cv * v[t];
            P1[t + 1] = P1[t] + cv;
            P2[t + 1] = P2[t] + cvv;
            C[t + 1] = C[t] + cnt[t];
        }
        prev.assign(m + 1, DBL_MAX);
        cur.assign(m + 1, DBL_MAX);
        arg.assign((size_t)(ke + 1) * (m + 1), 0);
        for (int i = 1; i <= m; ++i) prev[i] = cost(0, i);
        for (int j = 2; j <= ke; ++j) {
            std::fill(cur.begin(), cur.end(), DBL_MAX);
            if (j == ke) solve(j, m, m, j - 1, m - 1);  // only the full prefix is needed
            else solve(j, j, m, j - 1, m - 1);
            std::swap(prev, cur);
        }
        breaks[ke] = m;
        for (int j = ke; j >= 2; --j) breaks[j - 1] = arg[(size_t)j * (m + 1) + breaks[j]];
        breaks[0] = 0;
        return ke;
    }
};

struct RowScratch {
    std::vector<float> u;
    std::vector<std::pair<float, int>> order;
    std::vector<double> uv, ucnt;
    std::vector<int> cls;
    Jenks jk;
};

void gf4_row(const float *w, int K, int g, uint8_t *qrow, uint16_t *srow, uint16_t *cbrow, RowScratch &S) {
    S.u.resize(K);
    if (g) {
        for (int gi = 0; gi < K / g; ++gi) {
            float amax = 0.f;
            for (int k = 0; k < g; ++k) amax = std::max(amax, std::fabs(w[gi * g + k]));
            uint16_t hb = double_to_half_bits((double)amax);
            float s = half_bits_to_float(hb);
            if (amax == 0.f || s == 0.f || !std::isfinite(s)) { hb = 0x3c00u; s = 1.f; }
            srow[gi] = hb;
            for (int k = 0; k < g; ++k) S.u[gi * g + k] = w[gi * g + k] / s;
        }
    } else {
        std::memcpy(S.u.data(), w, sizeof(float) * (size_t)K);
    }
    S.order.resize(K);
    for (int k = 0; k < K; ++k) S.order[k] = {S.u[k], k};
    std::sort(S.order.begin(), S.order.end(),
              [](const std::pair<float, int> &a, const std::pair<float, int> &b) { return a.first < b.first; });
    S.uv.clear(); S.ucnt.clear();
    S.cls.resize(K);  // index of the distinct value each sorted slot belongs to
    for (int i = 0; i < K; ++i) {
        if (i == 0 || S.order[i].first != S.order[i - 1].first) {
            S.uv.push_back((double)S.order[i].first + 0.0);  // -0.0 and +0.0 are one value: +0.0
            S.ucnt.push_back(1.0);
        } else {
            S.ucnt.back() += 1.0;
        }
        S.cls[i] = (int)S.uv.size() - 1;
    }
    const int m = (int)S.uv.size();
    int breaks[17];
    const int ke = S.jk.run(S.uv.data(), S.ucnt.data(), m, 16, breaks);
    // class of each distinct value, and the class means
    std::vector<uint8_t> cls_of_u(m);
    for (int c = 0; c < ke; ++c) {
        for (int t = breaks[c]; t < breaks[c + 1]; ++t) cls_of_u[t] = (uint8_t)c;
        const double mean = (S.jk.P1[breaks[c + 1]] - S.jk.P1[breaks[c]]) / (S.jk.C[breaks[c + 1]] - S.jk.C[breaks[c]]);
        cbrow[c] = double_to_half_bits(mean);
    }
    // A row with an exact zero keeps it: the class that holds the value 0 gets the entry 0.0 instead of its mean
    // (pruned weights dequantise to exactly zero, as mask * s * (Q + Theta) does in the reference's forward).  The
    // codebook stays ascending: the neighbouring means lie outside this class's own value range, which contains 0.
    {
        const auto it = std::lower_bound(S.uv.begin(), S.uv.end(), 0.0);
        if (it != S.uv.end() && *it == 0.0) cbrow[cls_of_u[(size_t)(it - S.uv.begin())]] = 0;
    }
    for (int c = ke; c < 16; ++c) cbrow[c] = cbrow[ke - 1];
    std::memset(qrow, 0, (size_t)stride_codes(K) / 2);
    for (int i = 0; i < K; ++i) put_code(qrow, S.order[i].second, cls_of_u[S.cls[i]]);
}

void fwht128_inplace(float *v) {
    for (int s = 1; s < 128; s <<= 1)
        for (int base = 0; base < 128; base += 2 * s)
            for (int i = base; i < base + s; ++i) {
                const float a = v[i], b = v[i + s];
                v[i] = a + b;
                v[i + s] = a - b;
            }
    const float sc = 0.08838834764831845f;
    for (int i = 0; i < 128; ++i) v[i] = v[i] * sc;
}

}  // namespace

extern "C" int jq_pack_e2m1_host(const float *W, int N, int K, int g, uint8_t *qweight, uint16_t *scales, int threads) {
    if (!W || !qweight || !scales) return JQ_ERR_NULL_PTR;
    if (N <= 0 || K <= 0 || g <= 0 || g % 32 || K % g) return JQ_ERR_BAD_SHAPE;
    const int rb = stride_codes(K) / 2, G = K / g;
    parallel_rows(N, threads, [&](int n) {
        const float *w = W + (size_t)n * K;
        uint8_t *q = qweight + (size_t)n * rb;
        std::memset(q, 0, (size_t)rb);
        for (int gi = 0; gi < G; ++gi) {
            float amax = 0.f;
            for (int k = 0; k < g; ++k) amax = std::max(amax, std::fabs(w[gi * g + k]));
            const float q6 = amax / 6.0f;
            uint16_t hb = double_to_half_bits((double)q6);
            float s = half_bits_to_float(hb);
            if (amax == 0.f || s == 0.f) { hb = 0x3c00u; s = 1.f; }
            if (std::isinf(s)) { hb = 0x7bffu; s = 65504.f; }   // absmax / 6 beyond fp16: largest finite scale, codes saturate
            scales[(size_t)n * G + gi] = hb;
            for (int k = 0; k < g; ++k) put_code(q, gi * g + k, e2m1_code(w[gi * g + k] / s));
        }
    });
    return JQ_OK;
}

extern "C" int jq_pack_gf4_host(const float *W, int N, int K, int g, uint8_t *qweight, uint16_t *scales,
                                uint16_t *codebook, int threads) {
    if (!W || !qweight || !codebook) return JQ_ERR_NULL_PTR;
    if (N <= 0 || K <= 0 || g < 0 || (g && (g % 32 || K % g))) return JQ_ERR_BAD_SHAPE;
    if (g && !scales) return JQ_ERR_NULL_PTR;
    const int rb = stride_codes(K) / 2, G = g ? K / g : 0;
    int T = threads > 0 ? threads : (int)std::thread::hardware_concurrency();
    if (T < 1) T = 1;
    std::vector<RowScratch> scratch((size_t)T);
    std::atomic<int> next(0);
    auto work = [&](int sl) {
        RowScratch &S = scratch[(size_t)sl];
        for (;;) {
            int n = next.fetch_add(1);
            if (n >= N) break;
            gf4_row(W + (size_t)n * K, K, g, qweight + (size_t)n * rb, g ? scales + (size_t)n * G : nullptr,
                    codebook + (size_t)n * 16, S);
        }
    };
    if (T > N) T = N;
    if (T == 1) { work(0); return JQ_OK; }
    std::vector<std::thread> pool;
    for (int t = 0; t < T; ++t) pool.emplace_back(work, t);
    for (auto &th : pool) th.join();
    return JQ_OK;
}

extern "C" int jq_rotate_weights_host(float *W, int N, int K, int block, int threads) {
    if (!W) return JQ_ERR_NULL_PTR;
    if (block != 128) return JQ_ERR_UNSUPPORTED;
    if (N <= 0 || K <= 0 || K % block) return JQ_ERR_BAD_SHAPE;
    parallel_rows(N, threads, [&](int n) {
        for (int b = 0; b < K / 128; ++b) fwht128_inplace(W + (size_t)n * K + (size_t)b * 128);
    });
    return JQ_OK;
}
