// CPU oracle for the attention hot path of argus-engine.
//
// TEST INFRASTRUCTURE ONLY. This file is a plain C++ restatement of the reference's own CPU
// algorithms. It is the checker the CUDA kernels are compared against and the timed CPU baseline.
// Nothing in the shipped library links, loads or calls it; only tests/, the smoke check and the
// benchmark's CPU-baseline leg may use it.
//
// Every function names the reference source (path inside the argus-engine tree : lines) whose
// arithmetic it follows. All math is IEEE binary32 with contraction disabled at compile time
// (-ffp-contract=off) so that the bit-exact parts (KIVI codec, container order, keep-set
// selection) match the reference's Rust, which never fuses a*b+c on its own. The AVX2 arm uses
// explicit FMA intrinsics exactly where the reference's intrinsics do.
//
// Parity pinning: the reference holds no golden byte vectors for this path; it is pinned by the
// reference's own known-answer tests (codec blocks with literal fields, hand-computed score
// reductions, keep-list literals, analytic prefill cases). tests/test_oracle_*.py re-state those.

#include <immintrin.h>
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

inline float h2f(uint16_t h) { return _cvtsh_ss(h); }
inline uint16_t f2h(float f) { return _cvtss_sh(f, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC); }

constexpr float NEG_INF = -std::numeric_limits<float>::infinity();

// Element (kv, t, d) of a K/V tensor given element strides; covers both layouts of
// engine/src/kv/kv_cache.rs:238-266 (SeqMajor: pos*Hkv*D + h*D, HeadMajor: h*cap*D + pos*D).
struct KvView {
    const void* base;
    int is_f16;
    long head_stride;
    long pos_stride;
    inline float at(long kv, long t, long d) const {
        long off = kv * head_stride + t * pos_stride + d;
        return is_f16 ? h2f(static_cast<const uint16_t*>(base)[off])
                      : static_cast<const float*>(base)[off];
    }
};

}  // namespace

extern "C" {

// ───────────────────────────── conversions / data generators ─────────────────────────────

void orc_f32_to_f16(const float* src, uint16_t* dst, long n) {
    for (long i = 0; i < n; ++i) dst[i] = f2h(src[i]);
}
void orc_f16_to_f32(const uint16_t* src, float* dst, long n) {
    for (long i = 0; i < n; ++i) dst[i] = h2f(src[i]);
}

// Linear congruential test-data generator of the reference's unit tests
// (engine/src/backend/cpu/x86.rs:1546-1554): s = s*1103515245 + 12345 (wrapping u32),
// value = (i16)(s >> 16) / 32768.
void orc_lcg_gen(float* dst, long n, uint32_t seed) {
    uint32_t s = seed;
    for (long i = 0; i < n; ++i) {
        s = s * 1103515245u + 12345u;
        dst[i] = static_cast<float>(static_cast<int16_t>(s >> 16)) / 32768.0f;
    }
}

// ───────────────────────────── A1/A2: single-query GQA decode ─────────────────────────────
//
// Canonical three-pass form of Backend::attention_gen (engine/src/backend.rs:332-403):
// logits = (q·k)*scale in increasing d, max, exp(s-max), divide by the sum, then
// out += p_t * v_t in increasing t. `guards` adds the CPU backends' extras
// (engine/src/backend/cpu/common.rs:555-584): NaN logit -> -inf, all -inf or a bad sum -> uniform 1/T.
// scores (nullable) receives p_t at scores[h*score_stride + t].
int orc_attention_gen(const float* q, const void* k, const void* v, int kv_is_f16, float* out,
                      int hq, int hkv, int d, long T, long head_stride, long pos_stride,
                      float* scores, long score_stride, int guards) {
    if (hq <= 0 || hkv <= 0 || d <= 0 || T < 0 || hq % hkv) return -1;
    const KvView K{k, kv_is_f16, head_stride, pos_stride};
    const KvView V{v, kv_is_f16, head_stride, pos_stride};
    const float scale = 1.0f / std::sqrt(static_cast<float>(d));
    const int g = hq / hkv;
#pragma omp parallel for schedule(dynamic)
    for (int h = 0; h < hq; ++h) {
        const int kv = h / g;
        const float* qv = q + static_cast<long>(h) * d;
        std::vector<float> s(T);
        for (long t = 0; t < T; ++t) {
            float dot = 0.0f;
            for (int c = 0; c < d; ++c) dot += qv[c] * K.at(kv, t, c);
            s[t] = dot * scale;
        }
        if (guards)
            for (long t = 0; t < T; ++t)
                if (std::isnan(s[t])) s[t] = NEG_INF;
        float mx = NEG_INF;
        for (long t = 0; t < T; ++t) mx = std::fmax(mx, s[t]);
        bool uniform = false;
        if (guards && mx == NEG_INF) uniform = true;
        if (!uniform) {
            float sum = 0.0f;
            for (long t = 0; t < T; ++t) {
                s[t] = std::exp(s[t] - mx);
                sum += s[t];
            }
            if (guards && (std::isnan(sum) || sum <= 0.0f || std::isinf(sum))) uniform = true;
            else
                for (long t = 0; t < T; ++t) s[t] /= sum;
        }
        if (uniform) {
            const float u = 1.0f / static_cast<float>(T);
            for (long t = 0; t < T; ++t) s[t] = u;
        }
        if (scores)
            for (long t = 0; t < T; ++t) scores[static_cast<long>(h) * score_stride + t] = s[t];
        float* o = out + static_cast<long>(h) * d;
        for (int c = 0; c < d; ++c) o[c] = 0.0f;
        for (long t = 0; t < T; ++t) {
            const float w = s[t];
            for (int c = 0; c < d; ++c) o[c] += w * V.at(kv, t, c);
        }
    }
    return 0;
}

}  // extern "C"

// ───────────────────────────── A3: the AVX2 arm (timed CPU baseline) ─────────────────────────────
namespace {

// 8-lane exp: range reduction by ln2 split in two constants and a degree-5 minimax polynomial,
// 2^n through the exponent field (engine/src/backend/cpu/x86.rs:1269-1318).
inline __m256 exp8(__m256 x) {
    const __m256 hi = _mm256_set1_ps(88.3762626647949f);
    const __m256 lo = _mm256_set1_ps(-88.3762626647949f);
    x = _mm256_max_ps(_mm256_min_ps(x, hi), lo);
    __m256 n = _mm256_round_ps(_mm256_mul_ps(x, _mm256_set1_ps(1.44269504088896341f)),
                               _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC);
    __m256 r = _mm256_fnmadd_ps(n, _mm256_set1_ps(0.693359375f), x);
    r = _mm256_fnmadd_ps(n, _mm256_set1_ps(-2.12194440e-4f), r);
    const __m256 r2 = _mm256_mul_ps(r, r);
    __m256 p = _mm256_set1_ps(1.9875691500e-4f);
    p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(1.3981999507e-3f));
    p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(8.3334519073e-3f));
    p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(4.1665795894e-2f));
    p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(1.6666665459e-1f));
    p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(5.0000001201e-1f));
    p = _mm256_fmadd_ps(p, r2, r);
    p = _mm256_add_ps(p, _mm256_set1_ps(1.0f));
    const __m256i e = _mm256_slli_epi32(
        _mm256_add_epi32(_mm256_cvtps_epi32(n), _mm256_set1_epi32(127)), 23);
    return _mm256_mul_ps(p, _mm256_castsi256_ps(e));
}

inline float hsum8(__m256 v) {
    __m128 s = _mm_add_ps(_mm256_extractf128_ps(v, 1), _mm256_castps256_ps128(v));
    s = _mm_add_ps(s, _mm_movehl_ps(s, s));
    s = _mm_add_ss(s, _mm_movehdup_ps(s));
    return _mm_cvtss_f32(s);
}
inline float hmax8(__m256 v) {
    __m128 s = _mm_max_ps(_mm256_extractf128_ps(v, 1), _mm256_castps256_ps128(v));
    s = _mm_max_ps(s, _mm_movehl_ps(s, s));
    s = _mm_max_ss(s, _mm_movehdup_ps(s));
    return _mm_cvtss_f32(s);
}

// f32 · f16 dot with four 8-lane FMA accumulators over 32-element strides, then 8-element
// and scalar tails (engine/src/backend/cpu/x86.rs:608-666).
inline float dot_f32_f16(int n, const float* a, const uint16_t* b) {
    __m256 acc[4] = {_mm256_setzero_ps(), _mm256_setzero_ps(), _mm256_setzero_ps(),
                     _mm256_setzero_ps()};
    int i = 0;
    for (; i + 32 <= n; i += 32)
        for (int u = 0; u < 4; ++u) {
            __m256 bv = _mm256_cvtph_ps(
                _mm_loadu_si128(reinterpret_cast<const __m128i*>(b + i + 8 * u)));
            acc[u] = _mm256_fmadd_ps(_mm256_loadu_ps(a + i + 8 * u), bv, acc[u]);
        }
    for (; i + 8 <= n; i += 8) {
        __m256 bv = _mm256_cvtph_ps(_mm_loadu_si128(reinterpret_cast<const __m128i*>(b + i)));
        acc[0] = _mm256_fmadd_ps(_mm256_loadu_ps(a + i), bv, acc[0]);
    }
    float s = hsum8(_mm256_add_ps(_mm256_add_ps(acc[0], acc[1]), _mm256_add_ps(acc[2], acc[3])));
    for (; i < n; ++i) s += a[i] * h2f(b[i]);
    return s;
}
inline float dot_f32_f32(int n, const float* a, const float* b) {
    __m256 acc = _mm256_setzero_ps();
    int i = 0;
    for (; i + 8 <= n; i += 8)
        acc = _mm256_fmadd_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i), acc);
    float s = hsum8(acc);
    for (; i < n; ++i) s += a[i] * b[i];
    return s;
}

// out += w * f16 row (engine/src/backend/cpu/x86.rs:676-724).
inline void axpy_f16(int n, float* out, const uint16_t* v, float w) {
    const __m256 wv = _mm256_set1_ps(w);
    int i = 0;
    for (; i + 8 <= n; i += 8) {
        __m256 x = _mm256_cvtph_ps(_mm_loadu_si128(reinterpret_cast<const __m128i*>(v + i)));
        _mm256_storeu_ps(out + i, _mm256_fmadd_ps(wv, x, _mm256_loadu_ps(out + i)));
    }
    for (; i < n; ++i) out[i] += w * h2f(v[i]);
}
inline void axpy_f32(int n, float* out, const float* v, float w) {
    const __m256 wv = _mm256_set1_ps(w);
    int i = 0;
    for (; i + 8 <= n; i += 8)
        _mm256_storeu_ps(out + i,
                         _mm256_fmadd_ps(wv, _mm256_loadu_ps(v + i), _mm256_loadu_ps(out + i)));
    for (; i < n; ++i) out[i] += w * v[i];
}

// Row softmax: vector max, exp8(x-max) with a running vector sum, multiply by 1/sum
// (engine/src/backend/cpu/x86.rs:1477-1530). No NaN guard, as in the reference.
inline void softmax_row_avx2(float* p, long n) {
    __m256 mv = _mm256_set1_ps(NEG_INF);
    long i = 0;
    for (; i + 8 <= n; i += 8) mv = _mm256_max_ps(mv, _mm256_loadu_ps(p + i));
    float mx = hmax8(mv);
    for (; i < n; ++i) mx = std::fmax(mx, p[i]);
    const __m256 mxv = _mm256_set1_ps(mx);
    __m256 sv = _mm256_setzero_ps();
    for (i = 0; i + 8 <= n; i += 8) {
        __m256 e = exp8(_mm256_sub_ps(_mm256_loadu_ps(p + i), mxv));
        _mm256_storeu_ps(p + i, e);
        sv = _mm256_add_ps(sv, e);
    }
    float sum = hsum8(sv);
    for (; i < n; ++i) {
        p[i] = std::exp(p[i] - mx);
        sum += p[i];
    }
    const float inv = 1.0f / sum;
    const __m256 iv = _mm256_set1_ps(inv);
    for (i = 0; i + 8 <= n; i += 8) _mm256_storeu_ps(p + i, _mm256_mul_ps(_mm256_loadu_ps(p + i), iv));
    for (; i < n; ++i) p[i] *= inv;
}

}  // namespace

extern "C" {

// CpuBackendAVX2::attention_gen (engine/src/backend/cpu/x86.rs:178-357): one task per query
// head (the reference uses rayon par_chunks_mut(head_dim)); each task walks its KV head's rows,
// so K/V are re-read g times. n_threads<=0 means "all usable cores".
int orc_attention_gen_avx2(const float* q, const void* k, const void* v, int kv_is_f16, float* out,
                           int hq, int hkv, int d, long T, long head_stride, long pos_stride,
                           float* scores, long score_stride, int n_threads) {
    if (hq <= 0 || hkv <= 0 || d <= 0 || T < 0 || hq % hkv) return -1;
    const float scale = 1.0f / std::sqrt(static_cast<float>(d));
    const int g = hq / hkv;
#ifdef _OPENMP
    if (n_threads <= 0) n_threads = omp_get_max_threads();
#pragma omp parallel for schedule(dynamic) num_threads(n_threads)
#endif
    for (int h = 0; h < hq; ++h) {
        const int kv = h / g;
        const float* qv = q + static_cast<long>(h) * d;
        std::vector<float> s(T);
        if (kv_is_f16) {
            const uint16_t* kb = static_cast<const uint16_t*>(k) + kv * head_stride;
            for (long t = 0; t < T; ++t) s[t] = dot_f32_f16(d, qv, kb + t * pos_stride) * scale;
        } else {
            const float* kb = static_cast<const float*>(k) + kv * head_stride;
            for (long t = 0; t < T; ++t) s[t] = dot_f32_f32(d, qv, kb + t * pos_stride) * scale;
        }
        softmax_row_avx2(s.data(), T);
        if (scores) std::memcpy(scores + static_cast<long>(h) * score_stride, s.data(), T * sizeof(float));
        float* o = out + static_cast<long>(h) * d;
        for (int c = 0; c < d; ++c) o[c] = 0.0f;
        if (kv_is_f16) {
            const uint16_t* vb = static_cast<const uint16_t*>(v) + kv * head_stride;
            for (long t = 0; t < T; ++t) axpy_f16(d, o, vb + t * pos_stride, s[t]);
        } else {
            const float* vb = static_cast<const float*>(v) + kv * head_stride;
            for (long t = 0; t < T; ++t) axpy_f32(d, o, vb + t * pos_stride, s[t]);
        }
    }
    return 0;
}

int orc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// ───────────────────────────── A2 (prefill): tiled causal flash attention ─────────────────────────────
//
// flash_attention_head (engine/src/layers/attention.rs:78-221): row tiles of br, key tiles of bc,
// key c visible to row r iff c <= r + q_start (and c + window > r + q_start when window > 0),
// per-row online softmax (m, l, o) with alpha = 0 when the old max is -inf, final o / l (0 if l==0).
static void prefill_head(const float* q, long q_stride, const float* k, long k_stride,
                         const float* v, long v_stride, float* out, long out_stride, long q_len,
                         long kv_len, int d, long q_start, int br, int bc, long window) {
    const float scale = 1.0f / std::sqrt(static_cast<float>(d));
    std::vector<float> oi, li, mi, sij(bc), prow(bc);
    for (long r0 = 0; r0 < q_len; r0 += br) {
        const long r1 = std::min<long>(r0 + br, q_len);
        const long nb = r1 - r0;
        oi.assign(nb * d, 0.0f);
        li.assign(nb, 0.0f);
        mi.assign(nb, NEG_INF);
        for (long c0 = 0; c0 < kv_len; c0 += bc) {
            const long c1 = std::min<long>(c0 + bc, kv_len);
            const long nc = c1 - c0;
            if (c0 > (r1 - 1) + q_start) continue;
            if (window > 0 && c1 + window <= r0 + q_start + 1) continue;
            for (long r = 0; r < nb; ++r) {
                const long gq = r0 + r + q_start;
                float rmax = NEG_INF;
                bool any = false;
                for (long c = 0; c < nc; ++c) {
                    const long gc = c0 + c;
                    sij[c] = NEG_INF;
                    const bool ok = gc <= gq && (window <= 0 || gc + window > gq);
                    if (!ok) continue;
                    float dot = 0.0f;
                    const float* qp = q + (r0 + r) * q_stride;
                    const float* kp = k + gc * k_stride;
                    for (int e = 0; e < d; ++e) dot += qp[e] * kp[e];
                    const float val = dot * scale;
                    sij[c] = val;
                    if (val > rmax) rmax = val;
                    any = true;
                }
                if (!any) continue;
                const float m_prev = mi[r];
                const float m_new = std::fmax(m_prev, rmax);
                float lpart = 0.0f;
                for (long c = 0; c < nc; ++c) {
                    prow[c] = 0.0f;
                    if (sij[c] != NEG_INF) {
                        prow[c] = std::exp(sij[c] - m_new);
                        lpart += prow[c];
                    }
                }
                const float alpha = (m_prev == NEG_INF) ? 0.0f : std::exp(m_prev - m_new);
                li[r] = li[r] * alpha + lpart;
                mi[r] = m_new;
                for (int e = 0; e < d; ++e) {
                    float pv = 0.0f;
                    for (long c = 0; c < nc; ++c) {
                        const long gc = c0 + c;
                        const bool ok = gc <= gq && (window <= 0 || gc + window > gq);
                        if (ok) pv += prow[c] * v[gc * v_stride + e];
                    }
                    oi[r * d + e] = oi[r * d + e] * alpha + pv;
                }
            }
        }
        for (long r = 0; r < nb; ++r) {
            const float inv = (li[r] == 0.0f) ? 0.0f : 1.0f / li[r];
            for (int e = 0; e < d; ++e) out[(r0 + r) * out_stride + e] = oi[r * d + e] * inv;
        }
    }
}

// flash_attention_forward_strided over heads (engine/src/layers/attention.rs:233-351) and over
// the batch as prefill_attention drives it (engine/src/kv/standard_format.rs:1262-1310):
// Q/O [B,S,Hq,D]; K/V F32 with (k_pos_stride, kv_head_stride) = (D, cap*D) HeadMajor or
// (Hkv*D, D) SeqMajor, batch stride cap*Hkv*D; q_start = T - S. `bh_begin/bh_end` restrict the
// (batch*Hq) range so that a benchmark can time a stated subset.
int orc_flash_prefill(const float* q, const float* k, const float* v, float* out, int B, int hq,
                      int hkv, long S, long T, int d, long cap, int head_major, int br, int bc,
                      long window, long bh_begin, long bh_end, int n_threads) {
    if (hq <= 0 || hkv <= 0 || hq % hkv || T < S) return -1;
    const int g = hq / hkv;
    const long kps = head_major ? d : static_cast<long>(hkv) * d;
    const long khs = head_major ? cap * d : d;
    if (bh_end <= 0) bh_end = static_cast<long>(B) * hq;
#ifdef _OPENMP
    if (n_threads <= 0) n_threads = omp_get_max_threads();
#pragma omp parallel for schedule(dynamic) num_threads(n_threads)
#endif
    for (long bh = bh_begin; bh < bh_end; ++bh) {
        const long b = bh / hq, h = bh % hq;
        const float* qb = q + b * S * hq * d + h * d;
        float* ob = out + b * S * hq * d + h * d;
        const float* kb = k + b * cap * hkv * d + (h / g) * khs;
        const float* vb = v + b * cap * hkv * d + (h / g) * khs;
        prefill_head(qb, static_cast<long>(hq) * d, kb, kps, vb, kps, ob, static_cast<long>(hq) * d, S,
                     T, d, T - S, br, bc, window);
    }
    return 0;
}

// ───────────────────────────── A3: KIVI block codecs ─────────────────────────────
//
// BlockQ2_0 / BlockKVQ4 / BlockKVQ8 (crates/argus-kv-codec/src/lib.rs:36-73,125-157,175-202).
// 32 values -> {f16 d, f16 m, codes}; d = (max-min)/L with L = 3|15|255 in F32, id = d==0 ? 0 : 1/d,
// code = (u8)clamp(round((x-min)*id), 0, L) with round = half away from zero and NaN -> 0 (Rust `as u8`).
// Codes use the un-rounded F32 d; the stored d is its F16 rounding.
static inline int block_bytes(int bits) { return bits == 2 ? 12 : bits == 4 ? 20 : bits == 8 ? 36 : -1; }

static void quantize_block(const float* x, int bits, uint8_t* dst) {
    float mn = std::numeric_limits<float>::infinity(), mx = NEG_INF;
    for (int i = 0; i < 32; ++i) {
        mn = std::fmin(mn, x[i]);
        mx = std::fmax(mx, x[i]);
    }
    const float L = bits == 2 ? 3.0f : bits == 4 ? 15.0f : 255.0f;
    const float dd = (mx - mn) / L;
    const float id = (dd == 0.0f) ? 0.0f : 1.0f / dd;
    uint8_t code[32];
    for (int i = 0; i < 32; ++i) {
        float r = std::round((x[i] - mn) * id);
        r = std::isnan(r) ? 0.0f : std::fmin(std::fmax(r, 0.0f), L);
        code[i] = static_cast<uint8_t>(r);
    }
    const uint16_t d16 = f2h(dd), m16 = f2h(mn);
    std::memcpy(dst, &d16, 2);
    std::memcpy(dst + 2, &m16, 2);
    uint8_t* qs = dst + 4;
    if (bits == 8) {
        std::memcpy(qs, code, 32);
    } else if (bits == 4) {
        for (int i = 0; i < 16; ++i) qs[i] = static_cast<uint8_t>(code[2 * i] | (code[2 * i + 1] << 4));
    } else {
        for (int i = 0; i < 8; ++i)
            qs[i] = static_cast<uint8_t>(code[4 * i] | (code[4 * i + 1] << 2) | (code[4 * i + 2] << 4) |
                                         (code[4 * i + 3] << 6));
    }
}

static void dequantize_block(const uint8_t* src, int bits, float* out) {
    uint16_t d16, m16;
    std::memcpy(&d16, src, 2);
    std::memcpy(&m16, src + 2, 2);
    const float dd = h2f(d16), mm = h2f(m16);
    const uint8_t* qs = src + 4;
    for (int i = 0; i < 32; ++i) {
        unsigned c = bits == 8 ? qs[i] : bits == 4 ? ((qs[i / 2] >> ((i % 2) * 4)) & 0xF)
                                                   : ((qs[i / 4] >> ((i % 4) * 2)) & 0x3);
        out[i] = static_cast<float>(c) * dd + mm;
    }
}

int orc_kv_block_bytes(int bits) { return block_bytes(bits); }

int orc_kv_quantize(const float* src, long n_blocks, int bits, uint8_t* dst) {
    const int bb = block_bytes(bits);
    if (bb < 0) return -1;
    for (long b = 0; b < n_blocks; ++b) quantize_block(src + 32 * b, bits, dst + bb * b);
    return 0;
}
int orc_kv_dequantize(const uint8_t* src, long n_blocks, int bits, float* dst) {
    const int bb = block_bytes(bits);
    if (bb < 0) return -1;
    for (long b = 0; b < n_blocks; ++b) dequantize_block(src + bb * b, bits, dst + 32 * b);
    return 0;
}

// ───────────────────────────── A4: KIVI container (ring, flush order, view) ─────────────────────────────
//
// QuantizedRecentWindowCache (engine/src/kv/quant_window_cache.rs): update :2518-2562 appends
// tokens to the F32 ring [Hkv][res_cap][D], flushing first when the ring is full; flush_residual
// :844-965 pushes K blocks `for h, for group, for ch` (32 tokens of one channel) and V blocks
// `for h, for tok, for blk` (32 channels of one token); assemble_view :1463-1553 rebuilds the F32
// SeqMajor [T][Hkv][D] view.
struct OrcKivi {
    int hkv, d, res_cap, bits;
    long q_tokens = 0, res_pos = 0;
    std::vector<float> res_k, res_v;
    std::vector<uint8_t> qk, qv;
};

void* orc_kivi_new(int hkv, int d, int res_cap, int bits) {
    if (hkv <= 0 || d <= 0 || d % 32 || res_cap <= 0 || res_cap % 32 || block_bytes(bits) < 0)
        return nullptr;
    auto* c = new OrcKivi{hkv, d, res_cap, bits};
    c->res_k.assign(static_cast<size_t>(hkv) * res_cap * d, 0.0f);
    c->res_v.assign(static_cast<size_t>(hkv) * res_cap * d, 0.0f);
    return c;
}
void orc_kivi_free(void* p) { delete static_cast<OrcKivi*>(p); }

static void kivi_flush(OrcKivi* c) {
    const int bb = block_bytes(c->bits);
    const long n_groups = c->res_pos / 32, flush_tokens = n_groups * 32;
    float vals[32];
    uint8_t blk[36];
    for (int h = 0; h < c->hkv; ++h) {
        const long hb = static_cast<long>(h) * c->res_cap * c->d;
        for (long gi = 0; gi < n_groups; ++gi)
            for (int ch = 0; ch < c->d; ++ch) {
                for (int t = 0; t < 32; ++t) vals[t] = c->res_k[hb + (gi * 32 + t) * c->d + ch];
                quantize_block(vals, c->bits, blk);
                c->qk.insert(c->qk.end(), blk, blk + bb);
            }
    }
    for (int h = 0; h < c->hkv; ++h) {
        const long hb = static_cast<long>(h) * c->res_cap * c->d;
        for (long t = 0; t < flush_tokens; ++t)
            for (int b = 0; b < c->d / 32; ++b) {
                quantize_block(&c->res_v[hb + t * c->d + b * 32], c->bits, blk);
                c->qv.insert(c->qv.end(), blk, blk + bb);
            }
    }
    c->q_tokens += flush_tokens;
    const long remaining = c->res_pos - flush_tokens;
    if (remaining > 0)
        for (int h = 0; h < c->hkv; ++h) {
            const long hb = static_cast<long>(h) * c->res_cap * c->d;
            std::memmove(&c->res_k[hb], &c->res_k[hb + flush_tokens * c->d], remaining * c->d * 4);
            std::memmove(&c->res_v[hb], &c->res_v[hb + flush_tokens * c->d], remaining * c->d * 4);
        }
    c->res_pos = remaining;
}

// new_k/new_v: [seq_len][Hkv][D] F32 (SeqMajor), as the engine hands them to update().
int orc_kivi_update(void* p, const float* new_k, const float* new_v, long seq_len) {
    auto* c = static_cast<OrcKivi*>(p);
    for (long s = 0; s < seq_len; ++s) {
        if (c->res_pos >= c->res_cap) kivi_flush(c);
        for (int h = 0; h < c->hkv; ++h) {
            const long src = (s * c->hkv + h) * c->d;
            const long dst = (static_cast<long>(h) * c->res_cap + c->res_pos) * c->d;
            std::memcpy(&c->res_k[dst], new_k + src, c->d * 4);
            std::memcpy(&c->res_v[dst], new_v + src, c->d * 4);
        }
        c->res_pos += 1;
    }
    return 0;
}
long orc_kivi_q_tokens(void* p) { return static_cast<OrcKivi*>(p)->q_tokens; }
long orc_kivi_res_tokens(void* p) { return static_cast<OrcKivi*>(p)->res_pos; }
long orc_kivi_qk_bytes(void* p) { return static_cast<long>(static_cast<OrcKivi*>(p)->qk.size()); }
long orc_kivi_qv_bytes(void* p) { return static_cast<long>(static_cast<OrcKivi*>(p)->qv.size()); }
void orc_kivi_export(void* p, uint8_t* qk, uint8_t* qv, float* res_k, float* res_v) {
    auto* c = static_cast<OrcKivi*>(p);
    if (qk) std::memcpy(qk, c->qk.data(), c->qk.size());
    if (qv) std::memcpy(qv, c->qv.data(), c->qv.size());
    if (res_k) std::memcpy(res_k, c->res_k.data(), c->res_k.size() * 4);
    if (res_v) std::memcpy(res_v, c->res_v.data(), c->res_v.size() * 4);
}

// View assembly from raw buffers (so that it also serves buffers produced by the CUDA pack kernel).
// Writes K/V as F32 SeqMajor [T][Hkv][D], T = q_tokens + res_tokens.
int orc_kivi_assemble_view(const uint8_t* qk, const uint8_t* qv, const float* res_k, const float* res_v,
                           int hkv, int d, int res_cap, int bits, long q_tokens, long res_tokens,
                           float* view_k, float* view_v) {
    const int bb = block_bytes(bits);
    if (bb < 0 && q_tokens > 0) return -1;
    const long gpf = res_cap / 32, bpt = d / 32;
    const long n_flush = q_tokens / res_cap;
    long kb = 0, vb = 0;
    float buf[32];
    for (long f = 0; f < n_flush; ++f) {
        const long tok_base = f * res_cap;
        for (int h = 0; h < hkv; ++h)
            for (long gi = 0; gi < gpf; ++gi)
                for (int ch = 0; ch < d; ++ch) {
                    dequantize_block(qk + bb * kb++, bits, buf);
                    for (int t = 0; t < 32; ++t)
                        view_k[((tok_base + gi * 32 + t) * hkv + h) * d + ch] = buf[t];
                }
        for (int h = 0; h < hkv; ++h)
            for (long t = 0; t < res_cap; ++t)
                for (long b = 0; b < bpt; ++b) {
                    dequantize_block(qv + bb * vb++, bits, buf);
                    std::memcpy(&view_v[((tok_base + t) * hkv + h) * d + b * 32], buf, 128);
                }
    }
    for (int h = 0; h < hkv; ++h)
        for (long t = 0; t < res_tokens; ++t) {
            const long dst = ((q_tokens + t) * hkv + h) * d;
            const long src = (static_cast<long>(h) * res_cap + t) * d;
            std::memcpy(&view_k[dst], res_k + src, d * 4);
            std::memcpy(&view_v[dst], res_v + src, d * 4);
        }
    return 0;
}

// ───────────────────────────── A5: attention-score policy ─────────────────────────────
//
// One tracked layer of AttnScoreProducer::accumulate_layer_gqa
// (crates/techniques/attn-score/src/lib.rs:244-316): flat[t] = sum over q heads (h ascending),
// head[kv][t] = (sum over the g heads of the group) * (1/g); both combined into the step buffers
// with MAX at position score_offset + t.
void orc_score_accumulate_layer(const float* scores, long stride, long T, int hq, int hkv,
                                long score_offset, long max_seq, float* step_flat, float* step_head) {
    const long len = std::min(T, max_seq);
    const int g = hq / hkv;
    const float inv = 1.0f / static_cast<float>(g);
    for (long t = 0; t < len; ++t) {
        const long pos = score_offset + t;
        if (pos >= max_seq) break;
        float flat = 0.0f;
        for (int h = 0; h < hq; ++h) flat += scores[h * stride + t];
        step_flat[pos] = std::fmax(step_flat[pos], flat);
        if (!step_head) continue;
        for (int kv = 0; kv < hkv; ++kv) {
            float gs = 0.0f;
            for (int r = 0; r < g; ++r) gs += scores[(static_cast<long>(kv) * g + r) * stride + t];
            gs *= inv;
            step_head[kv * max_seq + pos] = std::fmax(step_head[kv * max_seq + pos], gs);
        }
    }
}

// begin_step decay + end_step add (same file :175-206, :318-359).
void orc_score_begin_step(float* importance, float* head_importance, float* step_flat, float* step_head,
                          int hkv, long max_seq, float decay) {
    if (decay > 0.0f) {
        const float f = 1.0f - decay;
        for (long i = 0; i < max_seq; ++i) importance[i] *= f;
        for (long i = 0; i < hkv * max_seq; ++i) head_importance[i] *= f;
    }
    std::fill(step_flat, step_flat + max_seq, 0.0f);
    std::fill(step_head, step_head + hkv * max_seq, 0.0f);
}
void orc_score_end_step(float* importance, float* head_importance, const float* step_flat,
                        const float* step_head, int hkv, long max_seq) {
    for (long i = 0; i < max_seq; ++i) importance[i] += step_flat[i];
    for (long i = 0; i < hkv * max_seq; ++i) head_importance[i] += step_head[i];
}

// The device-side twin of the same policy (crates/techniques/attn-score/src/score_reduce.cu:13-64):
// per token, MAX over layers of the head sum / group mean (starting from 0), then
// cumulative = cumulative*decay_factor + step.
void orc_score_fused_reduce(const float* scores, float* importance, float* head_importance,
                            float decay_factor, int n_layers, int hq, int hkv, long T,
                            long score_stride, long max_seq) {
    const int g = hq / hkv;
    const float inv = 1.0f / static_cast<float>(g);
    std::vector<float> lh(hkv), sh(hkv);
    for (long t = 0; t < T; ++t) {
        float sflat = 0.0f;
        std::fill(sh.begin(), sh.end(), 0.0f);
        for (int l = 0; l < n_layers; ++l) {
            float lf = 0.0f;
            std::fill(lh.begin(), lh.end(), 0.0f);
            for (int h = 0; h < hq; ++h) {
                const float w = scores[(static_cast<long>(l) * hq + h) * score_stride + t];
                lf += w;
                lh[h / g] += w;
            }
            sflat = std::fmax(sflat, lf);
            for (int kv = 0; kv < hkv; ++kv) sh[kv] = std::fmax(sh[kv], lh[kv] * inv);
        }
        importance[t] = importance[t] * decay_factor + sflat;
        for (int kv = 0; kv < hkv; ++kv)
            head_importance[kv * max_seq + t] = head_importance[kv * max_seq + t] * decay_factor + sh[kv];
    }
}
// Per-layer flat variant (score_reduce.cu:66-91): no cross-layer MAX.
void orc_score_reduce_per_layer(const float* scores, float* layer_flat, float decay_factor,
                                int n_layers, int hq, long T, long score_stride, long max_seq) {
    for (long t = 0; t < T; ++t)
        for (int l = 0; l < n_layers; ++l) {
            float s = 0.0f;
            for (int h = 0; h < hq; ++h) s += scores[(static_cast<long>(l) * hq + h) * score_stride + t];
            layer_flat[l * max_seq + t] = layer_flat[l * max_seq + t] * decay_factor + s;
        }
}

// ───────────────────────────── A6: keep-set selection ─────────────────────────────
//
// compile_keep_top_k (crates/argus-extension-api/src/lib.rs:788-810): prefix clamp, recent_start,
// STABLE descending sort of the middle by score with incomparable pairs (NaN) treated as equal,
// take `heavy`, ascending re-sort. Returns the keep count; keep must hold `current` entries.
long orc_keep_top_k(long current, long prefix, long recent, long heavy, const float* score,
                    long score_len, long* keep) {
    prefix = std::min(prefix, current);
    const long recent_start = std::max(current > recent ? current - recent : 0L, prefix);
    std::vector<std::pair<long, float>> mid;
    for (long p = prefix; p < recent_start; ++p)
        mid.emplace_back(p, (score && p < score_len) ? score[p] : 0.0f);
    // Rust's stable merge sort with a comparator that yields Equal for NaN pairs; std::stable_sort
    // with "a strictly greater than b" gives the same order whenever no NaN is present, which is
    // the only case the reference's tests (and ours) exercise.
    std::stable_sort(mid.begin(), mid.end(),
                     [](const std::pair<long, float>& a, const std::pair<long, float>& b) {
                         return a.second > b.second;
                     });
    std::vector<long> hv;
    for (long i = 0; i < static_cast<long>(mid.size()) && i < heavy; ++i) hv.push_back(mid[i].first);
    std::sort(hv.begin(), hv.end());
    long n = 0;
    for (long p = 0; p < prefix; ++p) keep[n++] = p;
    for (long p : hv) keep[n++] = p;
    for (long p = recent_start; p < current; ++p) keep[n++] = p;
    return n;
}

// H2O partition (crates/techniques/h2o/src/lib.rs:121-156): no-op (returns -1) while
// current <= prefix + hh + recent, else keep_top_k(current, prefix, recent, hh).
long orc_h2o_keep(long current, long protected_prefix, long hh_size, long recent_size,
                  const float* score, long score_len, long* keep) {
    const long prefix = std::min(protected_prefix, current);
    if (current <= prefix + hh_size + recent_size) return -1;
    if (!score) return orc_keep_top_k(current, prefix, hh_size + recent_size, 0, nullptr, 0, keep);
    return orc_keep_top_k(current, prefix, recent_size, hh_size, score, score_len, keep);
}

// ───────────────────────────── A7: merge of split partials ─────────────────────────────
//
// flash_merge_partials (engine/src/backend/cpu/neon.rs:1044-1125) in the (o, lse) form:
// partial c holds a normalised o_c[D] and lse_c = m_c + ln l_c; non-finite lse_c are skipped;
// out = sum exp(lse_c - M) o_c / sum exp(lse_c - M). Returns 0 when no partial was finite
// (the caller then owns the uniform fallback), else 1.
int orc_lse_merge(const float* o, const float* lse, int n_parts, int d, float* out) {
    float M = NEG_INF;
    for (int c = 0; c < n_parts; ++c)
        if (std::isfinite(lse[c]) && lse[c] > M) M = lse[c];
    for (int e = 0; e < d; ++e) out[e] = 0.0f;
    if (M == NEG_INF) return 0;
    float L = 0.0f;
    for (int c = 0; c < n_parts; ++c) {
        if (!std::isfinite(lse[c])) continue;
        const float a = std::exp(lse[c] - M);
        L += a;
        for (int e = 0; e < d; ++e) out[e] += a * o[c * d + e];
    }
    const float inv = 1.0f / L;
    for (int e = 0; e < d; ++e) out[e] *= inv;
    return 1;
}

}  // extern "C"
