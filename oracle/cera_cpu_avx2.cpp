// AVX2 + threads build of cera's x86 int8 GEMV/GEMM tier: the timed CPU baseline.
// TEST / BASELINE INFRASTRUCTURE ONLY - never linked into the CUDA library.
//
// Follows the AVX2 instantiation of the shared int8 kernel body
// (cera/src/backend/simd.rs:6306-6359: dot32u = maddubs + madd, dot32 = the sign
// trick; column tile 4).  Rows are split over a persistent spin-wait pool, the
// shape of the reference's RowPool (cera/src/backend/threadpool.rs:1-60).
// tests/test_oracle_avx2.py holds this bit-identical to the scalar restatement
// in cera_oracle.cpp.

#include "cera_oracle.h"

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstring>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

#if defined(__x86_64__)
#include <immintrin.h>
#define CERA_X86 1
#else
#define CERA_X86 0
#endif

namespace {

// ---- persistent row pool --------------------------------------------------
class RowPool {
  public:
    static RowPool &get() {
        // Leaked on purpose: parked workers still wait on the condition variable
        // at process exit, and destroying it under them would block.
        static RowPool *p = new RowPool();
        return *p;
    }
    // Runs f(lo, hi) over [0, m) split into `parts` contiguous ranges.
    void run(size_t m, int parts, const std::function<void(size_t, size_t)> &f) {
        if (parts <= 1 || m < 2) {
            f(0, m);
            return;
        }
        std::lock_guard<std::mutex> g(call_mu_);
        ensure(parts - 1);
        fn_ = &f;
        m_ = m;
        parts_ = parts;
        pending_.store(parts - 1, std::memory_order_relaxed);
        {
            std::lock_guard<std::mutex> lk(park_mu_);
            gen_.fetch_add(1, std::memory_order_release);
        }
        park_cv_.notify_all();
        span(0);
        while (pending_.load(std::memory_order_acquire) != 0) _mm_pause_compat();
    }

  private:
    static void _mm_pause_compat() {
#if CERA_X86
        _mm_pause();
#else
        std::this_thread::yield();
#endif
    }
    void span(int part) {
        const size_t per = (m_ + parts_ - 1) / parts_;
        const size_t lo = std::min(m_, per * (size_t)part), hi = std::min(m_, lo + per);
        if (lo < hi) (*fn_)(lo, hi);
    }
    void ensure(int n) {
        while ((int)workers_.size() < n) {
            const int id = (int)workers_.size() + 1;
            workers_.emplace_back([this, id] { loop(id); });
            workers_.back().detach();
        }
    }
    void loop(int id) {
        uint64_t seen = 0;
        for (;;) {
            uint64_t g;
            int spins = 0;
            while ((g = gen_.load(std::memory_order_acquire)) == seen) {
                if (++spins < 4000) {
                    _mm_pause_compat();
                } else {
                    // Park until the next call instead of burning a core.
                    std::unique_lock<std::mutex> lk(park_mu_);
                    park_cv_.wait(lk, [&] { return gen_.load(std::memory_order_acquire) != seen; });
                }
            }
            seen = g;
            if (id < parts_) {
                span(id);
                pending_.fetch_sub(1, std::memory_order_release);
            }
        }
    }
    std::mutex call_mu_, park_mu_;
    std::condition_variable park_cv_;
    std::vector<std::thread> workers_;
    std::atomic<uint64_t> gen_{0};
    std::atomic<int> pending_{0};
    const std::function<void(size_t, size_t)> *fn_ = nullptr;
    size_t m_ = 0;
    int parts_ = 1;
};

#if CERA_X86
// One source, two tiers (as the reference instantiates one kernel macro twice, cera/src/backend/simd.rs:6306-6359 and
// 7288-7345): the default build is the AVX2 tier; cera_cpu_vnni.cpp includes this file with CERA_TIER_VNNI defined,
// which swaps the 4-way byte dot for vpdpbusd (256-bit, AVX-512 VNNI + VL) and suffixes the entry points with _vnni.
#ifdef CERA_TIER_VNNI
#define TGT __attribute__((target("avx2,fma,f16c,avx512f,avx512vl,avx512vnni")))
#define CERA_CPU_FN(name) name##_vnni
#else
#define TGT __attribute__((target("avx2,fma,f16c")))
#define CERA_CPU_FN(name) name
#endif

// Integer-only half widen, inlined here so the per-block scale load costs no call
// (cera/src/quant.rs:48-73; tests compare it with cera_oracle_f16_to_f32).
inline float h2f_sw(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1Fu, mant = h & 0x3FFu;
    uint32_t rest;
    if (e == 0) {
        if (mant == 0) rest = 0;
        else {
            const uint32_t sh = (uint32_t)__builtin_clz(mant) - 21u;
            rest = ((113u - sh) << 23) | ((mant << (sh + 13u)) & 0x007FFFFFu);
        }
    } else if (e == 0x1F) rest = mant == 0 ? 0x7F800000u : (0x7FC00000u | (mant << 13));
    else rest = ((e + 112u) << 23) | (mant << 13);
    const uint32_t u = sign | rest;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline uint16_t rd16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

TGT inline __m256i dot32u(__m256i w, __m256i a) {
#ifdef CERA_TIER_VNNI
    return _mm256_dpbusd_epi32(_mm256_setzero_si256(), w, a);  // simd.rs:7305-7313; equal to the AVX2 form while no i16 saturates
#else
    return _mm256_madd_epi16(_mm256_maddubs_epi16(w, a), _mm256_set1_epi16(1));
#endif
}
TGT inline __m256i dot32s(__m256i w, __m256i a) {
    return dot32u(_mm256_sign_epi8(w, w), _mm256_sign_epi8(a, w));
}
TGT inline float hsum_ps(__m256 v) {
    __m128 s = _mm_add_ps(_mm256_extractf128_ps(v, 1), _mm256_castps256_ps128(v));
    s = _mm_add_ps(s, _mm_movehl_ps(s, s));
    return _mm_cvtss_f32(_mm_add_ss(s, _mm_shuffle_ps(s, s, 0x55)));
}
TGT inline int32_t hsum_i32(__m256i v) {
    __m128i s = _mm_add_epi32(_mm256_extracti128_si256(v, 1), _mm256_castsi256_si128(v));
    s = _mm_add_epi32(s, _mm_srli_si128(s, 8));
    s = _mm_add_epi32(s, _mm_srli_si128(s, 4));
    return _mm_cvtsi128_si32(s);
}
TGT inline __m256i ld256(const void *p) { return _mm256_loadu_si256((const __m256i *)p); }

constexpr int COLS = 4;  // column tile of the AVX2 instantiation

// Per-32-block and per-16-half activation sums (simd.rs:5651-5684).
TGT void col_sums(const int8_t *bq, size_t n, size_t k, std::vector<int32_t> &s32,
                  std::vector<int32_t> &s16, bool want16) {
    const size_t nb = k / 32;
    s32.resize(n * nb);
    if (want16) s16.resize(n * nb * 2);
    const __m256i ones = _mm256_set1_epi8(1);
    for (size_t j = 0; j < n; ++j)
        for (size_t b = 0; b < nb; ++b) {
            const __m256i p = dot32u(ones, ld256(bq + j * k + 32 * b));
            if (want16) {
                __m128i lo = _mm256_castsi256_si128(p), hi = _mm256_extracti128_si256(p, 1);
                lo = _mm_add_epi32(lo, _mm_srli_si128(lo, 8));
                lo = _mm_add_epi32(lo, _mm_srli_si128(lo, 4));
                hi = _mm_add_epi32(hi, _mm_srli_si128(hi, 8));
                hi = _mm_add_epi32(hi, _mm_srli_si128(hi, 4));
                s16[(j * nb + b) * 2] = _mm_cvtsi128_si32(lo);
                s16[(j * nb + b) * 2 + 1] = _mm_cvtsi128_si32(hi);
            }
            s32[j * nb + b] = hsum_i32(p);
        }
}

// ---- Q4_0 / Q8_0 ------------------------------------------------------------
template <bool Q4>
TGT void rows_q40_q80(const uint8_t *w, const float *bs, const int8_t *bq, float *out, size_t lo,
                      size_t hi, size_t n, size_t k) {
    const size_t nb = k / 32, bsz = Q4 ? 18 : 34, rb = nb * bsz;
    const __m128i m4 = _mm_set1_epi8(0x0F);
    for (size_t i = lo; i < hi; ++i) {
        const uint8_t *row = w + i * rb;
        for (size_t j0 = 0; j0 < n; j0 += COLS) {
            const int cols = (int)std::min<size_t>(COLS, n - j0);
            __m256 acc[COLS];
            for (int c = 0; c < COLS; ++c) acc[c] = _mm256_setzero_ps();
            for (size_t b = 0; b < nb; ++b) {
                const uint8_t *blk = row + b * bsz;
                __m256i wv;
                if (Q4) {
                    const __m128i qb = _mm_loadu_si128((const __m128i *)(blk + 2));
                    const __m128i l = _mm_and_si128(qb, m4);
                    const __m128i h = _mm_and_si128(_mm_srli_epi16(qb, 4), m4);
                    wv = _mm256_sub_epi8(_mm256_set_m128i(h, l), _mm256_set1_epi8(8));
                } else {
                    wv = ld256(blk + 2);
                }
                const float dw = h2f_sw(rd16(blk));
                for (int c = 0; c < cols; ++c) {
                    const size_t j = j0 + c;
                    const __m256 sc = _mm256_set1_ps(dw * bs[j * nb + b]);
                    acc[c] = _mm256_fmadd_ps(_mm256_cvtepi32_ps(dot32s(wv, ld256(bq + j * k + 32 * b))),
                                             sc, acc[c]);
                }
            }
            for (int c = 0; c < cols; ++c) out[i * n + j0 + c] = hsum_ps(acc[c]);
        }
    }
}

// ---- Q4_1 -------------------------------------------------------------------
TGT void rows_q4_1(const uint8_t *w, const float *bs, const int8_t *bq, const int32_t *cs, float *out,
                   size_t lo, size_t hi, size_t n, size_t k) {
    const size_t nb = k / 32, rb = nb * 20;
    const __m128i m4 = _mm_set1_epi8(0x0F);
    for (size_t i = lo; i < hi; ++i) {
        const uint8_t *row = w + i * rb;
        for (size_t j0 = 0; j0 < n; j0 += COLS) {
            const int cols = (int)std::min<size_t>(COLS, n - j0);
            __m256 acc[COLS];
            float macc[COLS] = {0, 0, 0, 0};
            for (int c = 0; c < COLS; ++c) acc[c] = _mm256_setzero_ps();
            for (size_t b = 0; b < nb; ++b) {
                const uint8_t *blk = row + b * 20;
                const float d = h2f_sw(rd16(blk)), mm = h2f_sw(rd16(blk + 2));
                const __m128i qb = _mm_loadu_si128((const __m128i *)(blk + 4));
                const __m256i wv = _mm256_set_m128i(_mm_and_si128(_mm_srli_epi16(qb, 4), m4),
                                                    _mm_and_si128(qb, m4));
                for (int c = 0; c < cols; ++c) {
                    const size_t j = j0 + c;
                    const float xs = bs[j * nb + b];
                    acc[c] = _mm256_fmadd_ps(_mm256_cvtepi32_ps(dot32u(wv, ld256(bq + j * k + 32 * b))),
                                             _mm256_set1_ps(xs * d), acc[c]);
                    macc[c] += xs * mm * (float)cs[j * nb + b];
                }
            }
            for (int c = 0; c < cols; ++c) out[i * n + j0 + c] = hsum_ps(acc[c]) + macc[c];
        }
    }
}

// 6-bit scale unpack (cera/src/quant.rs:591-605).
inline void kscales(const uint8_t *s, uint8_t sc[8], uint8_t mn[8]) {
    for (int j = 0; j < 4; ++j) {
        sc[j] = s[j] & 63;
        mn[j] = s[j + 4] & 63;
    }
    for (int j = 4; j < 8; ++j) {
        sc[j] = (uint8_t)((s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4));
        mn[j] = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

// ---- Q4_K -------------------------------------------------------------------
TGT void rows_q4_k(const uint8_t *w, const float *bs, const int8_t *bq, const int32_t *cs, float *out,
                   size_t lo, size_t hi, size_t n, size_t k) {
    const size_t sb = k / 256, nb = k / 32, rb = sb * 144;
    const __m256i m4 = _mm256_set1_epi8(0x0F);
    for (size_t i = lo; i < hi; ++i) {
        const uint8_t *row = w + i * rb;
        if (n == 1) {  // decode fast path: 4 round-robin chains
            __m256 f[4] = {_mm256_setzero_ps(), _mm256_setzero_ps(), _mm256_setzero_ps(),
                           _mm256_setzero_ps()};
            float macc = 0.0f;
            int slot = 0;
            for (size_t bi = 0; bi < sb; ++bi) {
                const uint8_t *blk = row + bi * 144;
                const float d = h2f_sw(rd16(blk)), dmin = h2f_sw(rd16(blk + 2));
                uint8_t sc[8], mn[8];
                kscales(blk + 4, sc, mn);
                for (int g = 0; g < 4; ++g) {
                    const __m256i qb = ld256(blk + 16 + 32 * g);
                    const __m256i wl = _mm256_and_si256(qb, m4);
                    const __m256i wh = _mm256_and_si256(_mm256_srli_epi16(qb, 4), m4);
                    for (int h = 0; h < 2; ++h) {
                        const int s = 2 * g + h;
                        const size_t xb = bi * 8 + s;
                        const float dsc = d * (float)sc[s], dmn = dmin * (float)mn[s];
                        const float xs = bs[xb];
                        f[slot] = _mm256_fmadd_ps(
                            _mm256_cvtepi32_ps(dot32u(h ? wh : wl, ld256(bq + 32 * xb))),
                            _mm256_set1_ps(xs * dsc), f[slot]);
                        macc += xs * dmn * (float)cs[xb];
                        slot = (slot + 1) & 3;
                    }
                }
            }
            out[i] = hsum_ps(_mm256_add_ps(_mm256_add_ps(f[0], f[1]), _mm256_add_ps(f[2], f[3]))) - macc;
            continue;
        }
        for (size_t j0 = 0; j0 < n; j0 += COLS) {
            const int cols = (int)std::min<size_t>(COLS, n - j0);
            __m256 acc[COLS];
            float macc[COLS] = {0, 0, 0, 0};
            for (int c = 0; c < COLS; ++c) acc[c] = _mm256_setzero_ps();
            for (size_t bi = 0; bi < sb; ++bi) {
                const uint8_t *blk = row + bi * 144;
                const float d = h2f_sw(rd16(blk)), dmin = h2f_sw(rd16(blk + 2));
                uint8_t sc[8], mn[8];
                kscales(blk + 4, sc, mn);
                for (int g = 0; g < 4; ++g) {
                    const __m256i qb = ld256(blk + 16 + 32 * g);
                    const __m256i wl = _mm256_and_si256(qb, m4);
                    const __m256i wh = _mm256_and_si256(_mm256_srli_epi16(qb, 4), m4);
                    for (int h = 0; h < 2; ++h) {
                        const int s = 2 * g + h;
                        const size_t xb = bi * 8 + s;
                        const float dsc = d * (float)sc[s], dmn = dmin * (float)mn[s];
                        for (int c = 0; c < cols; ++c) {
                            const size_t j = j0 + c;
                            const float xs = bs[j * nb + xb];
                            acc[c] = _mm256_fmadd_ps(
                                _mm256_cvtepi32_ps(dot32u(h ? wh : wl, ld256(bq + j * k + 32 * xb))),
                                _mm256_set1_ps(xs * dsc), acc[c]);
                            macc[c] += xs * dmn * (float)cs[j * nb + xb];
                        }
                    }
                }
            }
            for (int c = 0; c < cols; ++c) out[i * n + j0 + c] = hsum_ps(acc[c]) - macc[c];
        }
    }
}

// ---- Q6_K -------------------------------------------------------------------
TGT inline __m256i q6_group(const uint8_t *blk, int nh, int g) {
    const __m256i m4 = _mm256_set1_epi8(0x0F), m2 = _mm256_set1_epi8(0x03);
    const __m256i qlb = ld256(blk + nh * 64 + (g & 1) * 32);
    const __m256i qhb = ld256(blk + 128 + nh * 32);
    const __m256i l4 = g < 2 ? _mm256_and_si256(qlb, m4) : _mm256_and_si256(_mm256_srli_epi16(qlb, 4), m4);
    const __m256i h2 = _mm256_and_si256(_mm256_srl_epi16(qhb, _mm_cvtsi32_si128(2 * g)), m2);
    return _mm256_or_si256(l4, _mm256_slli_epi16(h2, 4));
}

TGT void rows_q6_k(const uint8_t *w, const float *bs, const int8_t *bq, const int32_t *cs16,
                   float *out, size_t lo, size_t hi, size_t n, size_t k) {
    const size_t sb = k / 256, nb = k / 32, rb = sb * 210;
    for (size_t i = lo; i < hi; ++i) {
        const uint8_t *row = w + i * rb;
        const bool fast = n == 1;
        for (size_t j0 = 0; j0 < n; j0 += fast ? 1 : COLS) {
            const int cols = fast ? 1 : (int)std::min<size_t>(COLS, n - j0);
            __m256 acc[COLS];
            float macc[COLS] = {0, 0, 0, 0};
            for (int c = 0; c < COLS; ++c) acc[c] = _mm256_setzero_ps();
            int slot = 0;
            for (size_t bi = 0; bi < sb; ++bi) {
                const uint8_t *blk = row + bi * 210;
                const int8_t *scales = (const int8_t *)(blk + 192);
                const float d = h2f_sw(rd16(blk + 208));
                const float d32 = d * 32.0f;
                for (int nh = 0; nh < 2; ++nh)
                    for (int g = 0; g < 4; ++g) {
                        const __m256i wv = q6_group(blk, nh, g);
                        const float sc0 = (float)scales[nh * 8 + 2 * g],
                                    sc1 = (float)scales[nh * 8 + 2 * g + 1];
                        const size_t xb = bi * 8 + nh * 4 + g;
                        const __m256 scd = _mm256_set_m128(_mm_set1_ps(sc1 * d), _mm_set1_ps(sc0 * d));
                        if (fast) {
                            const float xs = bs[xb];
                            acc[slot] = _mm256_fmadd_ps(
                                _mm256_cvtepi32_ps(dot32u(wv, ld256(bq + 32 * xb))),
                                _mm256_mul_ps(scd, _mm256_set1_ps(xs)), acc[slot]);
                            macc[0] += xs * d32 *
                                       (sc0 * (float)cs16[2 * xb] + sc1 * (float)cs16[2 * xb + 1]);
                            slot = (slot + 1) & 3;
                        } else {
                            for (int c = 0; c < cols; ++c) {
                                const size_t j = j0 + c;
                                const float xs = bs[j * nb + xb];
                                acc[c] = _mm256_fmadd_ps(
                                    _mm256_cvtepi32_ps(dot32u(wv, ld256(bq + j * k + 32 * xb))),
                                    _mm256_mul_ps(scd, _mm256_set1_ps(xs)), acc[c]);
                                macc[c] += xs * d32 * (sc0 * (float)cs16[(j * nb + xb) * 2] +
                                                       sc1 * (float)cs16[(j * nb + xb) * 2 + 1]);
                            }
                        }
                    }
            }
            if (fast) {
                out[i] = hsum_ps(_mm256_add_ps(_mm256_add_ps(acc[0], acc[1]),
                                               _mm256_add_ps(acc[2], acc[3]))) - macc[0];
            } else {
                for (int c = 0; c < cols; ++c) out[i * n + j0 + c] = hsum_ps(acc[c]) - macc[c];
            }
        }
    }
}
#endif  // CERA_X86

}  // namespace

extern "C" {

int CERA_CPU_FN(cera_cpu_has_avx2)(void) {
#if CERA_X86
#ifdef CERA_TIER_VNNI
    return __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma") && __builtin_cpu_supports("avx512vnni") &&
           __builtin_cpu_supports("avx512vl");
#else
    return __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
#endif
#else
    return 0;
#endif
}

int CERA_CPU_FN(cera_cpu_gemm_preq)(int type, const uint8_t *w, const float *bs, const int8_t *bq, float *out,
                                    size_t m, size_t n, size_t k, int n_threads) {
#if CERA_X86
    const bool kq = type == CERA_T_Q4_K || type == CERA_T_Q6_K;
    const bool ok = type == CERA_T_Q4_0 || type == CERA_T_Q8_0 || type == CERA_T_Q4_1 || kq;
    if (!CERA_CPU_FN(cera_cpu_has_avx2)() || !ok) return cera_oracle_gemm_preq(type, w, bs, bq, out, m, n, k);
    if (k % (kq ? 256 : 32)) return -1;
    std::vector<int32_t> s32, s16;
    if (type == CERA_T_Q4_1 || kq) col_sums(bq, n, k, s32, s16, type == CERA_T_Q6_K);
    const int parts = m >= 64 ? std::max(1, n_threads) : 1;
    RowPool::get().run(m, parts, [&](size_t lo, size_t hi) {
        switch (type) {
            case CERA_T_Q4_0: rows_q40_q80<true>(w, bs, bq, out, lo, hi, n, k); break;
            case CERA_T_Q8_0: rows_q40_q80<false>(w, bs, bq, out, lo, hi, n, k); break;
            case CERA_T_Q4_1: rows_q4_1(w, bs, bq, s32.data(), out, lo, hi, n, k); break;
            case CERA_T_Q4_K: rows_q4_k(w, bs, bq, s32.data(), out, lo, hi, n, k); break;
            case CERA_T_Q6_K: rows_q6_k(w, bs, bq, s16.data(), out, lo, hi, n, k); break;
        }
    });
    return 0;
#else
    (void)n_threads;
    return cera_oracle_gemm_preq(type, w, bs, bq, out, m, n, k);
#endif
}

int CERA_CPU_FN(cera_cpu_gemv)(int type, const uint8_t *w, const float *x, float *y, size_t m, size_t k,
                               int n_threads) {
    if (k % 32) return -1;
    std::vector<float> xs(k / 32);
    std::vector<int8_t> xq(k);
    cera_oracle_quantize_q8_0(x, k, xs.data(), xq.data());
    return CERA_CPU_FN(cera_cpu_gemm_preq)(type, w, xs.data(), xq.data(), y, m, 1, k, n_threads);
}

}  // extern "C"
