// CPU oracle for the TurboQuant KV-cache hot path. TEST INFRASTRUCTURE ONLY.
//
// This file restates, in plain scalar C++ with a C ABI, the arithmetic the
// reference project (fxslava/ascend-micro-harness) defines in its CPU golden
// models for the two operators this library accelerates:
//
//   * reshape_and_cache  (aligned 16-token writer, and the 1..16-token scatter
//     writer) -- rotation, power-of-two scale, signed INT4 codes, page layout;
//   * paged split-K decode attention -- query rotation, FP64 full-context and
//     per-split references, the log-sum-exp merge, the page partition.
//
// Every function cites the reference file:line it follows. Nothing here is
// used by the product path: only the test suite, the smoke check and the CPU
// baseline leg of the benchmark may call it. Parity of this restatement is
// pinned against the reference's own headers compiled in place (see
// ref_bridge.cpp) and against the committed golden vectors those produce.
//
// Build: g++ -O2 -std=c++17 -shared -fPIC -pthread tq_oracle.cpp -o libtq_oracle.so

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <thread>
#include <vector>

namespace {

constexpr int kGroup = 32;        // inner Hadamard width (tests/common/turboquant_oracle.hpp:51)
constexpr int kStrip = 16;        // strip height R (tests/common/turboquant_scatter_oracle.hpp:49)
constexpr float kMasked = -3.0e38f;  // kernels/ops/turboquant/turboquant_decode_tail.hpp:72

inline int parity(unsigned v) { return __builtin_popcount(v) & 1; }
// H[i][j] = (-1)^popcount(i & j)  (tests/common/turboquant_oracle.hpp:68-72)
inline int hsign(int i, int j) { return parity(static_cast<unsigned>(i & j)) ? -1 : 1; }

inline float bf16_to_f32(std::uint16_t raw)
{
    const std::uint32_t bits = static_cast<std::uint32_t>(raw) << 16;
    float v;
    std::memcpy(&v, &bits, 4);
    return v;
}

inline float half_to_f32(std::uint16_t h)
{
    const std::uint32_t sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu;
    std::uint32_t bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int e = -1;
            std::uint32_t m = man;
            do { ++e; m <<= 1; } while (!(m & 0x400u));
            bits = sign | static_cast<std::uint32_t>(127 - 15 - e) << 23 | (m & 0x3ffu) << 13;
        }
    } else if (exp == 31) bits = sign | 0x7f800000u | man << 13;
    else bits = sign | (exp + 112u) << 23 | man << 13;
    float v;
    std::memcpy(&v, &bits, 4);
    return v;
}
// Round-to-nearest-even narrowing (tests/common/turboquant_scatter_oracle.hpp:64-71).
inline std::uint16_t f32_to_bf16(float value)
{
    std::uint32_t bits;
    std::memcpy(&bits, &value, 4);
    if ((bits & 0x7f800000u) == 0x7f800000u && (bits & 0x7fffffu))
        return static_cast<std::uint16_t>((bits >> 16) | 0x40u);
    return static_cast<std::uint16_t>((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
}

// y = M x with M = (H_G (x) I32) diag(s) (I_G (x) H32), un-normalised, in the
// factored order of tests/common/turboquant_oracle.hpp:382-410. T is long long
// for the integer writer and double for non-integer bf16 activations.
template <class T>
void rotate_factored(int d, const int* signs, const T* x, T* y)
{
    const int groups = d / kGroup;
    std::vector<T> z(static_cast<std::size_t>(d));
    for (int g = 0; g < groups; ++g)
        for (int o = 0; o < kGroup; ++o) {
            T acc = 0;
            for (int i = 0; i < kGroup; ++i) acc += static_cast<T>(hsign(o, i)) * x[g * kGroup + i];
            z[g * kGroup + o] = acc;
        }
    for (int c1 = 0; c1 < groups; ++c1)
        for (int c0 = 0; c0 < kGroup; ++c0) {
            T acc = 0;
            for (int g = 0; g < groups; ++g) {
                const int ch = g * kGroup + c0;
                acc += static_cast<T>(hsign(c1, g) * signs[ch]) * z[ch];
            }
            y[c1 * kGroup + c0] = acc;
        }
}

// The radix-2 cascade of tests/common/rotate_butterfly_oracle.hpp:130-142 in
// FP32: stage s computes out[i] = in[i^s] + ((i&s) ? -in[i] : in[i]).
// ingress (y = Pi x): strides 1..16, sign diagonal, strides 32..d/2.
// egress  (y = x Pi): strides 32..d/2, sign diagonal, strides 1..16.
void butterfly_f32(int d, const float* signs, const float* x, float* y, bool ingress,
                   float scale)
{
    std::vector<float> v(x, x + d), n(static_cast<std::size_t>(d));
    auto stage = [&](int s) {
        for (int i = 0; i < d; ++i) n[i] = v[i ^ s] + ((i & s) ? -v[i] : v[i]);
        v.swap(n);
    };
    auto sign = [&]() {
        for (int i = 0; i < d; ++i) v[i] *= signs[i];
    };
    if (ingress) {
        for (int s = 1; s < kGroup; s <<= 1) stage(s);
        sign();
        for (int s = kGroup; s < d; s <<= 1) stage(s);
    } else {
        for (int s = kGroup; s < d; s <<= 1) stage(s);
        sign();
        for (int s = 1; s < kGroup; s <<= 1) stage(s);
    }
    for (int i = 0; i < d; ++i) y[i] = v[i] * scale;
}

// Round half to even of y / 2^shift (tests/common/turboquant_oracle.hpp:100-111).
long long rint_even_shift(long long y, int shift)
{
    if (shift <= 0) return y << (-shift);
    const long long den = 1LL << shift;
    long long q = y / den;
    const long long rem = y % den;
    if (rem == 0) return q;
    const long long twice = 2 * (rem < 0 ? -rem : rem);
    if (twice > den || (twice == den && (q % 2 != 0))) q += (y >= 0 ? 1 : -1);
    return q;
}

inline void put_nibble(std::uint8_t* base, std::size_t index, int q)
{
    const std::uint8_t nib = static_cast<std::uint8_t>(q & 0xF);
    std::uint8_t& b = base[index / 2];
    b = (index % 2 == 0) ? static_cast<std::uint8_t>((b & 0xF0u) | nib)
                         : static_cast<std::uint8_t>((b & 0x0Fu) | (nib << 4));
}

inline int get_nibble(const std::uint8_t* base, std::size_t index)
{
    const int raw = (base[index / 2] >> ((index % 2) * 4)) & 15;
    return raw >= 8 ? raw - 16 : raw;
}

// Power-of-two quantiser for one rotated row held as exact integers
// (tests/common/turboquant_oracle.hpp:412-439). floor_at_one selects the
// aligned writer's absmax floor; without it an all-zero row takes the scatter
// writer's branch scale = 1, codes 0
// (tests/common/turboquant_scatter_oracle.hpp:192-200).
void quantise_int_row(int d, const long long* y, float inv_sqrt_len, bool floor_at_one, int* q,
                      float* scale)
{
    long long m = floor_at_one ? 1 : 0;
    for (int c = 0; c < d; ++c) m = std::max(m, y[c] < 0 ? -y[c] : y[c]);
    if (m == 0) {
        *scale = 1.0f;
        for (int c = 0; c < d; ++c) q[c] = 0;
        return;
    }
    int e = 0;
    while ((1LL << (e + 1)) <= m) ++e;
    *scale = std::ldexp(1.0f, e - 2) * inv_sqrt_len;
    for (int c = 0; c < d; ++c) {
        long long v = rint_even_shift(y[c], e - 2);
        q[c] = static_cast<int>(v > 7 ? 7 : v);
    }
}

// The same quantiser for a non-integer FP32 row: the exponent comes from the
// FP32 bit pattern of absmax and the product y * 2^(2-e) is exact, so one
// round-half-even is the only rounding
// (kernels/ops/turboquant/turboquant_reshape_and_cache_a8.cpp:1136-1158,:1207-1209).
void quantise_f32_row(int d, const float* y, float inv_sqrt_len, bool floor_at_one, int* q,
                      float* scale)
{
    float m = floor_at_one ? 1.0f : 0.0f;
    for (int c = 0; c < d; ++c) m = std::fmax(m, std::fabs(y[c]));
    if (m == 0.0f) {
        *scale = 1.0f;
        for (int c = 0; c < d; ++c) q[c] = 0;
        return;
    }
    const int e = std::ilogb(m);
    *scale = std::ldexp(1.0f, e - 2) * inv_sqrt_len;
    for (int c = 0; c < d; ++c) {
        const double scaled = std::fmin(std::ldexp(static_cast<double>(y[c]), 2 - e), 7.0);
        q[c] = static_cast<int>(std::nearbyint(scaled));
    }
}

template <class F>
void parallel_for(int n, int threads, F&& body)
{
    if (threads <= 1 || n <= 1) {
        for (int i = 0; i < n; ++i) body(i);
        return;
    }
    threads = std::min(threads, n);
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t)
        pool.emplace_back([&, t]() {
            for (int i = t; i < n; i += threads) body(i);
        });
    for (auto& th : pool) th.join();
}

struct Geometry {
    int H, d, S, P;
    std::size_t head_bytes() const { return static_cast<std::size_t>(S) * d / 2; }
    std::size_t key_nibble(int page, int head, int tok, int ch) const
    {  // tests/common/turboquant_scatter_oracle.hpp:107-112
        return ((static_cast<std::size_t>(page) * H + head) * S + tok) * d + ch;
    }
    std::size_t value_nibble(int page, int head, int tok, int ch) const
    {  // tests/common/turboquant_scatter_oracle.hpp:114-124
        return (static_cast<std::size_t>(page) * H + head) * S * d +
               static_cast<std::size_t>(tok / kStrip) * (kStrip * d) +
               static_cast<std::size_t>(ch) * kStrip + tok % kStrip;
    }
    std::size_t scale_index(int plane, int page, int head, int tok) const
    {  // tests/common/turboquant_oracle.hpp:342-346
        return ((static_cast<std::size_t>(plane) * P + page) * H + head) * S + tok;
    }
};

// One input element as the exact value the device reads.
inline double load_act(int dtype, const void* base, std::size_t index)
{
    if (dtype == 0) return static_cast<const std::int8_t*>(base)[index];
    return bf16_to_f32(static_cast<const std::uint16_t*>(base)[index]);
}

bool row_is_integer(int d, const double* x)
{
    for (int c = 0; c < d; ++c)
        if (x[c] != std::nearbyint(x[c]) || std::fabs(x[c]) > 32768.0) return false;
    return true;
}

// Rotate + quantise one (token, head, plane) row into codes and a scale.
void process_row(int dtype, const void* src, std::size_t row_offset, int d, const int* signs,
                 float inv_sqrt_len, bool floor_at_one, int* q, float* scale)
{
    std::vector<double> x(static_cast<std::size_t>(d));
    for (int c = 0; c < d; ++c) x[c] = load_act(dtype, src, row_offset + c);
    if (row_is_integer(d, x.data())) {
        std::vector<long long> xi(static_cast<std::size_t>(d)), yi(static_cast<std::size_t>(d));
        for (int c = 0; c < d; ++c) xi[c] = static_cast<long long>(x[c]);
        rotate_factored<long long>(d, signs, xi.data(), yi.data());
        quantise_int_row(d, yi.data(), inv_sqrt_len, floor_at_one, q, scale);
        return;
    }
    // Non-integer bf16 activations: the rotation is evaluated in FP64 (exact
    // for bf16 operands of comparable exponent) and narrowed once to FP32, the
    // type the device accumulates in. Not bit-pinned by the reference: its
    // validation only demands bit equality for integer-valued inputs
    // (tests/npu/validation/test_turboquant_bf16_validation.cpp:3-17).
    std::vector<double> y(static_cast<std::size_t>(d));
    rotate_factored<double>(d, signs, x.data(), y.data());
    std::vector<float> yf(static_cast<std::size_t>(d));
    for (int c = 0; c < d; ++c) yf[c] = static_cast<float>(y[c]);
    quantise_f32_row(d, yf.data(), inv_sqrt_len, floor_at_one, q, scale);
}

}  // namespace

extern "C" {

// ---------------------------------------------------------------- rotation
// Resident rotation blocks T[s][g][c0][i] = (s?-1:1) signs[g*32+c0] H32[c0][i]
// (tests/common/turboquant_oracle.hpp:157-171). out holds 2*(d/32) blocks.
void tqo_build_tables_i8(int d, const int* signs, std::int8_t* out)
{
    const int groups = d / kGroup;
    for (int s = 0; s < 2; ++s)
        for (int g = 0; g < groups; ++g)
            for (int c0 = 0; c0 < kGroup; ++c0)
                for (int i = 0; i < kGroup; ++i)
                    out[((static_cast<std::size_t>(s) * groups + g) * kGroup + c0) * kGroup + i] =
                        static_cast<std::int8_t>((s ? -1 : 1) * signs[g * kGroup + c0] *
                                                 hsign(c0, i));
}

// Writer fixture sign diagonal (tests/common/turboquant_oracle.hpp:77-80).
int tqo_pi_sign_writer(int channel)
{
    return ((channel * channel + 3 * channel + 1) % 7 < 3) ? -1 : 1;
}

// Decode fixture sign diagonal (tests/common/paged_decode_oracle.hpp:148-152).
int tqo_pi_sign_decode(int channel)
{
    const unsigned x = static_cast<unsigned>(channel);
    return ((x * 2654435761u) >> 13) & 1u ? -1 : 1;
}

void tqo_rotate_int(int d, const int* signs, const long long* x, long long* y)
{
    rotate_factored<long long>(d, signs, x, y);
}

// Dense definition of the same matrix, for the factorisation self-check
// (tests/cpu/test_reshape_and_cache_a8_probe.cpp:150-167).
void tqo_rotate_dense_int(int d, const int* signs, const long long* x, long long* y)
{
    for (int r = 0; r < d; ++r) {
        long long acc = 0;
        for (int c = 0; c < d; ++c)
            acc += static_cast<long long>(hsign(r / kGroup, c / kGroup) *
                                          signs[(c / kGroup) * kGroup + r % kGroup] *
                                          hsign(r % kGroup, c % kGroup)) * x[c];
        y[r] = acc;
    }
}

void tqo_butterfly_f32(int d, const float* signs, const float* x, float* y, int ingress,
                       float scale)
{
    butterfly_f32(d, signs, x, y, ingress != 0, scale);
}

// Query rotation as the decode path defines it: q_rot = bf16(Pi q), Pi = M/sqrt(d)
// (tests/common/paged_decode_oracle.hpp:481-514). Evaluated as the FP32 ingress
// cascade followed by one multiply, so the result is reproducible bit for bit.
void tqo_rotate_query_bf16(int rows, int d, const float* signs, float inv_sqrt_len,
                           const std::uint16_t* q, std::uint16_t* q_rot)
{
    std::vector<float> x(static_cast<std::size_t>(d)), y(static_cast<std::size_t>(d));
    for (int r = 0; r < rows; ++r) {
        for (int c = 0; c < d; ++c) x[c] = bf16_to_f32(q[static_cast<std::size_t>(r) * d + c]);
        butterfly_f32(d, signs, x.data(), y.data(), true, inv_sqrt_len);
        for (int c = 0; c < d; ++c) q_rot[static_cast<std::size_t>(r) * d + c] = f32_to_bf16(y[c]);
    }
}

// ------------------------------------------------------- aligned writer
// tq_oracle::compute_oracle_reference (tests/common/turboquant_oracle.hpp:476-513)
// with the slot contract of page_of_slots (:278-287). dtype 0 = int8, 1 = bf16.
// Caches are updated in place for the pages a strip owns; page_written (may be
// null) receives one flag per page. Returns the first strip that violates the
// slot contract, or -1.
int tqo_reshape_and_cache(int dtype, const void* key, const void* value,
                          const std::int32_t* slots, const int* signs, int T, int H, int d,
                          int S, int P, float inv_sqrt_len, std::uint8_t* key_cache,
                          std::uint8_t* value_cache, float* scale_cache,
                          std::uint8_t* page_written, int threads)
{
    // The reference's writer fixes the page at one strip (S = 16); a page of S = 16 k tokens
    // holds k strips, each at a strip boundary of its page (the in-page offset of the
    // project's later aligned-prefill design).
    if (T <= 0 || H <= 0 || S <= 0 || S % kStrip != 0 || d % kGroup != 0 || T % kStrip != 0) return -2;
    const Geometry g{H, d, S, P};
    const int strips = T / kStrip;
    std::vector<int> slot_of(static_cast<std::size_t>(strips), -1);
    int bad = -1;
    for (int s = 0; s < strips; ++s) {
        const std::int32_t* ss = slots + static_cast<std::size_t>(s) * kStrip;
        bool ok = ss[0] >= 0 && ss[0] % kStrip == 0;
        for (int i = 1; ok && i < kStrip; ++i) ok = ss[i] == ss[0] + i;
        if (ok && ss[0] / S < P) slot_of[s] = ss[0];
        else if (bad < 0) bad = s;
    }
    parallel_for(strips, threads, [&](int s) {
        if (slot_of[s] < 0) return;
        const int page = slot_of[s] / S, tip = slot_of[s] % S;
        if (page_written) page_written[page] = 1;
        std::vector<int> q(static_cast<std::size_t>(d));
        for (int plane = 0; plane < 2; ++plane) {
            const void* src = plane == 0 ? key : value;
            std::uint8_t* cache = plane == 0 ? key_cache : value_cache;
            for (int head = 0; head < H; ++head)
                for (int t = 0; t < kStrip; ++t) {
                    const std::size_t row =
                        (static_cast<std::size_t>(s) * kStrip + t) * H * d + static_cast<std::size_t>(head) * d;
                    float scale;
                    process_row(dtype, src, row, d, signs, inv_sqrt_len, true, q.data(), &scale);
                    for (int c = 0; c < d; ++c)
                        put_nibble(cache, plane == 0 ? g.key_nibble(page, head, tip + t, c)
                                                     : g.value_nibble(page, head, tip + t, c), q[c]);
                    scale_cache[g.scale_index(plane, page, head, tip + t)] = scale;
                }
        }
    });
    return bad;
}

// ------------------------------------------------- aligned writer, ragged requests
// The aligned writer over requests of any length (the project's design note for it:
// reports/qwen35_turboquant_rfc.md:564-650): request b owns tokens cu_seqlens[b] ..
// cu_seqlens[b+1]; its strips never straddle a request boundary; the last strip of a
// request may hold n < 16 tokens. For such a strip the key plane receives n rows and the
// scale planes n entries; the value plane receives the whole channel-major strip with the
// missing tokens as zeros (a partial channel-major strip is not a contiguous region).
// Each strip's slots must be consecutive and start on a strip boundary of a page.
// bf16 input. Returns the number of strips that broke the slot contract.
int tqo_reshape_and_cache_varlen(const std::uint16_t* key, const std::uint16_t* value,
                                 const std::int32_t* slots, const int* signs,
                                 const std::int32_t* cu_seqlens, int num_requests, int H, int d,
                                 int S, int P, float inv_sqrt_len, std::uint8_t* key_cache,
                                 std::uint8_t* value_cache, float* scale_cache)
{
    if (S % kStrip != 0 || d % kGroup != 0) return -2;
    const Geometry g{H, d, S, P};
    std::vector<int> q(static_cast<std::size_t>(d));
    int bad = 0;
    for (int b = 0; b < num_requests; ++b) {
        const int begin = cu_seqlens[b], len = cu_seqlens[b + 1] - begin;
        for (int r = 0; r * kStrip < len; ++r) {
            const int t0 = begin + r * kStrip, n = std::min(kStrip, len - r * kStrip);
            const std::int32_t slot0 = slots[t0];
            bool ok = slot0 >= 0 && slot0 % kStrip == 0 && slot0 / S < P;
            for (int i = 1; ok && i < n; ++i) ok = slots[t0 + i] == slot0 + i;
            if (!ok) { ++bad; continue; }
            const int page = slot0 / S, tip = slot0 % S;
            for (int plane = 0; plane < 2; ++plane) {
                const std::uint16_t* src = plane == 0 ? key : value;
                std::uint8_t* cache = plane == 0 ? key_cache : value_cache;
                for (int head = 0; head < H; ++head)
                    for (int t = 0; t < kStrip; ++t) {
                        if (t < n) {
                            const std::size_t row = static_cast<std::size_t>(t0 + t) * H * d +
                                                    static_cast<std::size_t>(head) * d;
                            float scale;
                            process_row(1, src, row, d, signs, inv_sqrt_len, true, q.data(), &scale);
                            scale_cache[g.scale_index(plane, page, head, tip + t)] = scale;
                        } else if (plane == 0) {
                            continue;            // key rows past the tail stay as they were
                        } else {
                            std::fill(q.begin(), q.end(), 0);   // value strip: zero padding
                        }
                        for (int c = 0; c < d; ++c)
                            put_nibble(cache, plane == 0 ? g.key_nibble(page, head, tip + t, c)
                                                         : g.value_nibble(page, head, tip + t, c), q[c]);
                    }
            }
        }
    }
    return bad;
}

// ------------------------------------------------------- scatter writer
// tq_scatter::compute_reference (tests/common/turboquant_scatter_oracle.hpp:291-342)
// over the run discovery of the device kernel
// (kernels/ops/turboquant/turboquant_reshape_scatter_aiv.cpp:693-730):
// request r owns tokens cu_seqlens[r]..cu_seqlens[r+1] (or token r when
// cu_seqlens is null), slot < 0 is a padded token, every other nibble and
// scale of the caches is preserved. key/value are bf16 [tokens][H*d].
int tqo_reshape_scatter(const std::uint16_t* key, const std::uint16_t* value,
                        const std::int32_t* slots, const float* signs_f,
                        const std::int32_t* cu_seqlens, int num_requests, int H, int d, int S,
                        int P, float inv_sqrt_len, std::uint8_t* key_cache,
                        std::uint8_t* value_cache, float* scale_cache)
{
    if (S % kStrip != 0 || d % kGroup != 0) return -2;
    const Geometry g{H, d, S, P};
    std::vector<int> q(static_cast<std::size_t>(d));
    std::vector<float> x(static_cast<std::size_t>(d)), y(static_cast<std::size_t>(d));
    for (int r = 0; r < num_requests; ++r) {
        const int begin = cu_seqlens ? cu_seqlens[r] : r;
        const int end = cu_seqlens ? cu_seqlens[r + 1] : r + 1;
        for (int tok = begin; tok < end; ++tok) {
            const int slot = slots[tok];
            if (slot < 0) continue;
            const int page = slot / S, tib = slot % S;
            if (page >= P) return -3;
            for (int head = 0; head < H; ++head)
                for (int plane = 0; plane < 2; ++plane) {
                    const std::size_t row =
                        static_cast<std::size_t>(tok) * H * d + static_cast<std::size_t>(head) * d;
                    // quantise_row (tests/common/turboquant_scatter_oracle.hpp:185-217):
                    // the FP32 ingress cascade, then the quantiser with no absmax floor.
                    const std::uint16_t* src = plane == 0 ? key : value;
                    for (int c = 0; c < d; ++c) x[c] = bf16_to_f32(src[row + c]);
                    butterfly_f32(d, signs_f, x.data(), y.data(), true, 1.0f);
                    float scale;
                    quantise_f32_row(d, y.data(), inv_sqrt_len, false, q.data(), &scale);
                    std::uint8_t* cache = plane == 0 ? key_cache : value_cache;
                    for (int c = 0; c < d; ++c)
                        put_nibble(cache, plane == 0 ? g.key_nibble(page, head, tib, c)
                                                     : g.value_nibble(page, head, tib, c), q[c]);
                    scale_cache[g.scale_index(plane, page, head, tib)] = scale;
                }
        }
    }
    return 0;
}

// -------------------------------------------------------------- decode
// Page partition (include/turboquant_splitk_contract.hpp:129-136).
void tqo_partition(std::uint32_t pages, std::uint32_t splits, std::uint32_t split,
                   std::uint32_t* begin, std::uint32_t* count)
{
    const std::uint32_t width = (pages + splits - 1u) / splits;
    const std::uint32_t b = split * width;
    const std::uint32_t remaining = b < pages ? pages - b : 0u;
    *begin = b;
    *count = remaining < width ? remaining : width;
}

// FP64 softmax attention of one sequence over logical tokens [tok_begin, tok_end)
// clipped to ctx_len, reading the packed caches through the block table. This is
// splitk_decode_test::Fixture::Reference (tests/common/splitk_decode_fixture.hpp:193-248)
// and ReferenceAicPartial (tests/common/aic_splitk_decode_fixture.hpp:32-77) with
// runtime head_size, page size and query-row count:
//   score[t] = (sum_c q_rot[c] Kq[t][c]) kscale[t] softmax_scale
//   m = max score (-3e38 when the range holds no live token), l = sum exp(score-m)
//   acc[c] = sum_t exp(score-m) vscale[t] Vq[c][t]
// q_rot is bf16 [rows][d]; outputs are m[rows], l[rows], acc[rows][d] in FP64.
static void decode_partial_f32q(const float* q_rot, int rows, const std::uint8_t* key_cache,
                                const std::uint8_t* value_cache, const float* scale_cache,
                                const std::int32_t* block_table, int H, int head, int d, int S, int P,
                                int ctx_len, int tok_begin, int tok_end, float softmax_scale,
                                double* m, double* l, double* acc);
void tqo_decode_partial(const std::uint16_t* q_rot, int rows, const std::uint8_t* key_cache,
                        const std::uint8_t* value_cache, const float* scale_cache,
                        const std::int32_t* block_table, int H, int head, int d, int S, int P,
                        int ctx_len, int tok_begin, int tok_end, float softmax_scale, double* m,
                        double* l, double* acc)
{
    std::vector<float> qf(static_cast<std::size_t>(rows) * d);
    for (std::size_t i = 0; i < qf.size(); ++i) qf[i] = bf16_to_f32(q_rot[i]);
    decode_partial_f32q(qf.data(), rows, key_cache, value_cache, scale_cache, block_table, H, head, d, S,
                        P, ctx_len, tok_begin, tok_end, softmax_scale, m, l, acc);
}
static void decode_partial_f32q(const float* q_rot, int rows, const std::uint8_t* key_cache,
                                const std::uint8_t* value_cache, const float* scale_cache,
                                const std::int32_t* block_table, int H, int head, int d, int S, int P,
                                int ctx_len, int tok_begin, int tok_end, float softmax_scale,
                                double* m, double* l, double* acc)
{
    const Geometry g{H, d, S, P};
    const int hi = std::min(tok_end, ctx_len);
    std::vector<double> scores(static_cast<std::size_t>(std::max(0, hi - tok_begin)));
    for (int r = 0; r < rows; ++r) {
        m[r] = static_cast<double>(kMasked);
        l[r] = 0.0;
        for (int c = 0; c < d; ++c) acc[static_cast<std::size_t>(r) * d + c] = 0.0;
        for (int t = tok_begin; t < hi; ++t) {
            const int page = block_table[t / S], tib = t % S;
            double dot = 0.0;
            for (int c = 0; c < d; ++c)
                dot += static_cast<double>(q_rot[static_cast<std::size_t>(r) * d + c]) *
                       get_nibble(key_cache, g.key_nibble(page, head, tib, c));
            const double s = dot * scale_cache[g.scale_index(0, page, head, tib)] *
                             static_cast<double>(softmax_scale);
            scores[t - tok_begin] = s;
            m[r] = std::max(m[r], s);
        }
        for (int t = tok_begin; t < hi; ++t) {
            const int page = block_table[t / S], tib = t % S;
            const double p = std::exp(scores[t - tok_begin] - m[r]);
            l[r] += p;
            const double pv = p * scale_cache[g.scale_index(1, page, head, tib)];
            for (int c = 0; c < d; ++c)
                acc[static_cast<std::size_t>(r) * d + c] +=
                    pv * get_nibble(value_cache, g.value_nibble(page, head, tib, c));
        }
    }
}

// Log-sum-exp merge of partial states in FP64
// (routines/routine_probe_l2_atomic_sync.hpp:116-121; neutral element -3e38/0/0
// as in tests/cpu/test_splitk_decode_probe.cpp:48-61). state = {m, l, acc[d]}.
void tqo_lse_merge(int d, double* m, double* l, double* acc, double m2, double l2,
                   const double* acc2)
{
    const double mn = std::max(*m, m2);
    const double a = std::exp(*m - mn), b = std::exp(m2 - mn);
    *l = *l * a + l2 * b;
    for (int c = 0; c < d; ++c) acc[c] = acc[c] * a + acc2[c] * b;
    *m = mn;
}

// Whole decode for a batch: rotate q (bf16 [B][Hq][d]) once, attend over every
// live token, emit FP64 context [B][Hq][d].
//   output_stage 0: acc / l in the rotated basis
//   output_stage 1: (acc / l) Pi  -- the egress rotation, here as a dense FP64
//                   product (tests/common/single_token_decode_oracle.hpp:339-349)
//   output_stage 2: stage 1 divided by 1 + exp(-gate)
//                   (tests/common/paged_decode_oracle.hpp:598-617)
// block_tables is int32 [B][max_blocks]; context_lens int32 [B]; gate (may be
// null unless stage 2) FP32 [B][Hq][d]. A sequence with no live token yields 0.
// q_f16 = 0: bf16 query, rotation rounded to bf16 (the operand the reference pins);
// q_f16 = 1: FP16 query whose FP32 rotation is used as it is (the fused decoder keeps an FP32
// rotated image, include/turboquant_fused_decode_opt.hpp:160-169).
static void decode_impl(int q_f16, const std::uint16_t* q, const std::uint8_t* key_cache,
                        const std::uint8_t* value_cache, const float* scale_cache,
                        const std::int32_t* block_tables, const std::int32_t* context_lens,
                        const float* signs, const float* gate, int B, int Hq, int Hkv, int d, int S,
                        int P, int max_blocks, float inv_sqrt_len, float softmax_scale,
                        int output_stage, double* out, int threads)
{
    const int group = Hq / Hkv;
    parallel_for(B * Hkv, threads, [&](int item) {
        const int b = item / Hkv, kvh = item % Hkv;
        const std::uint16_t* qsrc = q + (static_cast<std::size_t>(b) * Hq + kvh * group) * d;
        std::vector<float> qrot(static_cast<std::size_t>(group) * d);
        if (q_f16) {
            std::vector<float> x(static_cast<std::size_t>(d));
            for (int r = 0; r < group; ++r) {
                for (int c = 0; c < d; ++c) x[c] = half_to_f32(qsrc[static_cast<std::size_t>(r) * d + c]);
                butterfly_f32(d, signs, x.data(), qrot.data() + static_cast<std::size_t>(r) * d, true, inv_sqrt_len);
            }
        } else {
            std::vector<std::uint16_t> bits(static_cast<std::size_t>(group) * d);
            tqo_rotate_query_bf16(group, d, signs, inv_sqrt_len, qsrc, bits.data());
            for (std::size_t i = 0; i < bits.size(); ++i) qrot[i] = bf16_to_f32(bits[i]);
        }
        std::vector<double> m(group), l(group), acc(static_cast<std::size_t>(group) * d);
        decode_partial_f32q(qrot.data(), group, key_cache, value_cache, scale_cache,
                            block_tables + static_cast<std::size_t>(b) * max_blocks, Hkv, kvh, d, S, P,
                            context_lens[b], 0, context_lens[b], softmax_scale, m.data(), l.data(),
                            acc.data());
        for (int r = 0; r < group; ++r) {
            double* o = out + (static_cast<std::size_t>(b) * Hq + kvh * group + r) * d;
            std::vector<double> n(static_cast<std::size_t>(d));
            for (int c = 0; c < d; ++c)
                n[c] = l[r] > 0.0 ? acc[static_cast<std::size_t>(r) * d + c] / l[r] : 0.0;
            if (output_stage == 0) {
                for (int c = 0; c < d; ++c) o[c] = n[c];
                continue;
            }
            for (int oc = 0; oc < d; ++oc) {
                double sum = 0.0;  // ctx[oc] = sum_c n[c] Pi[c][oc]
                for (int c = 0; c < d; ++c) {
                    const int c1 = c / kGroup, c0 = c % kGroup, gg = oc / kGroup, i = oc % kGroup;
                    sum += n[c] * (hsign(c1, gg) * hsign(c0, i)) *
                           static_cast<double>(signs[gg * kGroup + c0]);
                }
                sum *= static_cast<double>(inv_sqrt_len);
                if (output_stage == 2) {
                    const double gt = gate[(static_cast<std::size_t>(b) * Hq + kvh * group + r) * d + oc];
                    sum /= 1.0 + std::exp(-gt);
                }
                o[oc] = sum;
            }
        }
    });
}

void tqo_decode(const std::uint16_t* q, const std::uint8_t* key_cache,
                const std::uint8_t* value_cache, const float* scale_cache,
                const std::int32_t* block_tables, const std::int32_t* context_lens,
                const float* signs, const float* gate, int B, int Hq, int Hkv, int d, int S,
                int P, int max_blocks, float inv_sqrt_len, float softmax_scale, int output_stage,
                double* out, int threads)
{
    decode_impl(0, q, key_cache, value_cache, scale_cache, block_tables, context_lens, signs, gate, B, Hq,
                Hkv, d, S, P, max_blocks, inv_sqrt_len, softmax_scale, output_stage, out, threads);
}
void tqo_decode_f16q(const std::uint16_t* q, const std::uint8_t* key_cache,
                     const std::uint8_t* value_cache, const float* scale_cache,
                     const std::int32_t* block_tables, const std::int32_t* context_lens,
                     const float* signs, const float* gate, int B, int Hq, int Hkv, int d, int S,
                     int P, int max_blocks, float inv_sqrt_len, float softmax_scale,
                     int output_stage, double* out, int threads)
{
    decode_impl(1, q, key_cache, value_cache, scale_cache, block_tables, context_lens, signs, gate, B, Hq,
                Hkv, d, S, P, max_blocks, inv_sqrt_len, softmax_scale, output_stage, out, threads);
}

// ===================================================================== routines
// The single-purpose routines of the reference that the two operators above do not
// call, and the ingest/decode variant built from them (block-diagonal H16 rotation,
// RMS scale, 16-level Lloyd-Max codes).

// Y = X x H16 for 16x16 tiles, X FP16 row-major, H16[k][c] = (-1)^popcount(k & c),
// FP32 accumulation in k order (include/sim_micro_testbed.hpp:181-198).
void tqo_hadamard16(const std::uint16_t* x_f16, float* y, int tiles)
{
    for (int t = 0; t < tiles; ++t)
        for (int row = 0; row < 16; ++row)
            for (int col = 0; col < 16; ++col) {
                float sum = 0;
                for (int k = 0; k < 16; ++k)
                    sum += half_to_f32(x_f16[(t * 16 + row) * 16 + k]) * static_cast<float>(hsign(k, col));
                y[(t * 16 + row) * 16 + col] = sum;
            }
}

// 16-level Lloyd-Max codebook for N(0,1): Gaussian conditional-mean fixed point with
// midpoint thresholds (include/routines/routine_vector_lloydmax_quantize.hpp:18-30).
static const float kLmCentroids[16] = {
    -2.732589571f, -2.069017227f, -1.618046386f, -1.256231197f, -0.942340456f, -0.656759119f,
    -0.388048299f, -0.128395030f, 0.128395030f,  0.388048299f,  0.656759119f,  0.942340456f,
    1.256231197f,  1.618046386f,  2.069017227f,  2.732589571f};
static const float kLmThresholds[15] = {
    -2.400803399f, -1.843531806f, -1.437138792f, -1.099285827f, -0.799549788f, -0.522403709f,
    -0.258221665f, 0.f,           0.258221665f,  0.522403709f,  0.799549788f,  1.099285827f,
    1.437138792f,  1.843531806f,  2.400803399f};
// code = #{thresholds <= x}: equality goes to the upper bin (same header :32-38).
static inline unsigned lm_code(float x)
{
    unsigned q = 0;
    for (float t : kLmThresholds) q += x >= t;
    return q;
}
void tqo_lloydmax4_tables(float* centroids16, float* thresholds15)
{
    std::memcpy(centroids16, kLmCentroids, sizeof kLmCentroids);
    std::memcpy(thresholds15, kLmThresholds, sizeof kLmThresholds);
}
// codes packed low nibble first in element order (tests/common/lloydmax_oracle.hpp:65-69);
// recon (optional) = centroid of the code.
void tqo_lloydmax4_quantize(const float* x, std::uint8_t* packed, float* recon, long long n)
{
    for (long long i = 0; i < n; ++i) {
        const unsigned q = lm_code(x[i]);
        if ((i & 1) == 0) packed[i / 2] = static_cast<std::uint8_t>(q);
        else packed[i / 2] |= static_cast<std::uint8_t>(q << 4);
        if (recon) recon[i] = kLmCentroids[q];
    }
}

// y = 14 sigmoid(x) - 7 evaluated exactly in double, rounded once to nearest-even and
// saturated to [-8, 7]; byte j = element 2j low, 2j+1 high (tests/cpu/icdf_fixture.hpp:5-20).
void tqo_icdf_quantize(const std::uint16_t* x, int is_bf16, std::uint8_t* packed, long long n)
{
    for (long long i = 0; i < n; ++i) {
        const double v = is_bf16 ? bf16_to_f32(x[i]) : half_to_f32(x[i]);
        const double y = 14.0 / (1.0 + std::exp(-v)) - 7.0;
        int q = static_cast<int>(std::nearbyint(y));
        q = std::max(-8, std::min(7, q));
        const unsigned nib = static_cast<unsigned>(q) & 0xFu;
        if ((i & 1) == 0) packed[i / 2] = static_cast<std::uint8_t>(nib);
        else packed[i / 2] |= static_cast<std::uint8_t>(nib << 4);
    }
}

// ---- the writer built from those routines (the variant the project brief words as
// "block-diagonal 16x16 Sylvester Hadamard, per-token FP32 scale, 16-level Lloyd-Max"):
//   y     = x H16 per 16-channel block (integers stay exact), y_rot = y / 4
//   scale = sqrt(sum y_rot^2) * inv_sqrt_len + 1e-20
//           (kernels/ops/turboquant/baseline/common/turboquant_codec_950.h:194-207)
//   code  = lloydmax(y_rot * (1 / scale)), unsigned 0..15, low nibble first (the vendored codec
//           also multiplies by a reciprocal, same file :197-207)
// into the same planes as the power-of-two writer (key token-major, value channel-major
// per 16-token strip, planar FP32 scales). Every operation and its order is fixed (no fused
// multiply-add), so the kernel reproduces scale bits and codes for any finite input.
static void lm_token(const float* x, int d, float inv_sqrt_len, unsigned* codes, float* scale_out)
{
    // y = x H16 per block as the radix-2 butterfly (strides 1, 2, 4, 8), the order the kernel
    // uses; squares summed four at a time in FP32, the groups in FP64 per half of the channels
    std::vector<float> y(x, x + d), tmp(d);
    for (int s = 1; s < 16; s <<= 1) {
        for (int i = 0; i < d; ++i) tmp[i] = (i & s) ? y[i ^ s] - y[i] : y[i ^ s] + y[i];
        y = tmp;
    }
    double half[2] = {0, 0};
    for (int h = 0; h < 2; ++h)
        for (int g = h * (d / 8); g < (h + 1) * (d / 8); ++g) {
            volatile float q4 = y[4 * g] * y[4 * g];
            for (int i = 1; i < 4; ++i) {
                volatile float sq = y[4 * g + i] * y[4 * g + i];
                q4 = q4 + sq;
            }
            half[h] += static_cast<double>(q4);
        }
    const double s2 = half[0] + half[1];
    const float root = static_cast<float>(std::sqrt(s2));
    volatile float scaled = root * 0.25f;
    scaled = scaled * inv_sqrt_len;
    const float scale = scaled + 1e-20f;
    const float inv = 1.0f / scale;
    for (int c = 0; c < d; ++c) {
        volatile float yr = y[c] * 0.25f;
        codes[c] = lm_code(yr * inv);
    }
    *scale_out = scale;
}
int tqo_reshape_and_cache_lm(int dtype, const void* key, const void* value,
                             const std::int32_t* slots, int num_tokens, int H, int d, int S, int P,
                             float inv_sqrt_len, std::uint8_t* key_cache,
                             std::uint8_t* value_cache, float* scale_cache)
{
    if (num_tokens % kStrip || d % 16 || S % kStrip) return -1;
    int bad = 0;
    std::vector<float> x(d);
    std::vector<unsigned> codes(d);
    for (int strip = 0; strip < num_tokens / kStrip; ++strip) {
        const std::int32_t slot0 = slots[strip * kStrip];
        bool ok = slot0 >= 0 && slot0 % kStrip == 0 && slot0 / S < P;
        for (int i = 0; i < kStrip; ++i) ok = ok && slots[strip * kStrip + i] == slot0 + i;
        if (!ok) { ++bad; continue; }
        const std::size_t page = slot0 / S, tip = slot0 % S;
        for (int plane = 0; plane < 2; ++plane)
            for (int h = 0; h < H; ++h) {
                std::uint8_t* cache = plane ? value_cache : key_cache;
                const std::size_t head_base = (page * H + h) * static_cast<std::size_t>(S) * (d / 2);
                for (int t = 0; t < kStrip; ++t) {
                    const std::size_t row = (static_cast<std::size_t>(strip) * kStrip + t) * H * d +
                                            static_cast<std::size_t>(h) * d;
                    for (int c = 0; c < d; ++c)
                        x[c] = dtype == 0
                                   ? static_cast<float>(static_cast<const std::int8_t*>(plane ? value : key)[row + c])
                                   : bf16_to_f32(static_cast<const std::uint16_t*>(plane ? value : key)[row + c]);
                    float scale;
                    lm_token(x.data(), d, inv_sqrt_len, codes.data(), &scale);
                    scale_cache[((static_cast<std::size_t>(plane) * P + page) * H + h) * S + tip + t] = scale;
                    for (int c = 0; c < d; ++c) {
                        const std::size_t nib = plane == 0
                            ? (tip + t) * static_cast<std::size_t>(d) + c
                            : (tip / kStrip) * static_cast<std::size_t>(kStrip) * d + static_cast<std::size_t>(c) * kStrip + t;
                        std::uint8_t& byte = cache[head_base + nib / 2];
                        byte = (nib & 1) ? static_cast<std::uint8_t>((byte & 0x0F) | (codes[c] << 4))
                                         : static_cast<std::uint8_t>((byte & 0xF0) | codes[c]);
                    }
                }
            }
    }
    return bad;
}

// q_rot = bf16((q H16 per block) / 4), the FP32 butterfly over strides 1, 2, 4, 8 inside
// each 16-channel block (out[i] = in[i ^ s] + ((i & s) ? -in[i] : in[i])).
static void lm_rotate_block16(float* v, int d)
{
    std::vector<float> tmp(d);
    for (int s = 1; s < 16; s <<= 1) {
        for (int i = 0; i < d; ++i) tmp[i] = v[i ^ s] + ((i & s) ? -v[i] : v[i]);
        std::copy(tmp.begin(), tmp.end(), v);
    }
}
void tqo_lm_rotate_query_bf16(int rows, int d, const std::uint16_t* q, std::uint16_t* q_rot)
{
    std::vector<float> v(d);
    for (int r = 0; r < rows; ++r) {
        for (int c = 0; c < d; ++c) v[c] = bf16_to_f32(q[r * d + c]);
        lm_rotate_block16(v.data(), d);
        for (int c = 0; c < d; ++c) q_rot[r * d + c] = f32_to_bf16(v[c] * 0.25f);
    }
}

// FP64 decode over a Lloyd-Max cache: score = sum_c q_rot[c] centroid[K] * kscale * softmax_scale,
// acc += p * vscale * centroid[V], out = (acc / l) rotated back (output_stage 1) or not (0).
void tqo_decode_lm(const std::uint16_t* q, const std::uint8_t* key_cache,
                   const std::uint8_t* value_cache, const float* scale_cache,
                   const std::int32_t* block_tables, const std::int32_t* context_lens, int B, int Hq,
                   int Hkv, int d, int S, int P, int max_blocks, float softmax_scale,
                   int output_stage, double* out, int threads)
{
    const int G = Hq / Hkv;
    auto work = [&](int begin, int end) {
        std::vector<std::uint16_t> qr(d);
        std::vector<double> acc(d);
        std::vector<float> ctx(d);
        for (int item = begin; item < end; ++item) {
            const int b = item / Hq, hq = item % Hq, h = hq / G;
            tqo_lm_rotate_query_bf16(1, d, q + static_cast<std::size_t>(item) * d, qr.data());
            const int n = std::max(0, context_lens[b]);
            double m = -std::numeric_limits<double>::infinity(), l = 0;
            std::fill(acc.begin(), acc.end(), 0.0);
            for (int t = 0; t < n; ++t) {
                const std::size_t page = block_tables[static_cast<std::size_t>(b) * max_blocks + t / S];
                const int tip = t % S;
                const std::size_t head_base = (page * Hkv + h) * static_cast<std::size_t>(S) * (d / 2);
                double dot = 0;
                for (int c = 0; c < d; ++c) {
                    const std::size_t nib = static_cast<std::size_t>(tip) * d + c;
                    const unsigned code = (key_cache[head_base + nib / 2] >> (4 * (nib & 1))) & 0xF;
                    dot += static_cast<double>(bf16_to_f32(qr[c])) * kLmCentroids[code];
                }
                const double ks = scale_cache[((0 * static_cast<std::size_t>(P) + page) * Hkv + h) * S + tip];
                const double vs = scale_cache[((1 * static_cast<std::size_t>(P) + page) * Hkv + h) * S + tip];
                const double s = dot * ks * softmax_scale;
                const double mn = std::max(m, s), a = std::exp(m - mn), pw = std::exp(s - mn);
                l = l * a + pw;
                for (int c = 0; c < d; ++c) {
                    const std::size_t nib = static_cast<std::size_t>(tip / kStrip) * kStrip * d +
                                            static_cast<std::size_t>(c) * kStrip + tip % kStrip;
                    const unsigned code = (value_cache[head_base + nib / 2] >> (4 * (nib & 1))) & 0xF;
                    acc[c] = acc[c] * a + pw * vs * kLmCentroids[code];
                }
                m = mn;
            }
            for (int c = 0; c < d; ++c) ctx[c] = l > 0 ? static_cast<float>(acc[c] / l) : 0.f;
            if (output_stage == 1) {
                lm_rotate_block16(ctx.data(), d);
                for (int c = 0; c < d; ++c) ctx[c] *= 0.25f;
            }
            for (int c = 0; c < d; ++c) out[static_cast<std::size_t>(item) * d + c] = ctx[c];
        }
    };
    const int total = B * Hq;
    threads = std::max(1, std::min(threads, total));
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t)
        pool.emplace_back(work, static_cast<int>(static_cast<long long>(total) * t / threads),
                          static_cast<int>(static_cast<long long>(total) * (t + 1) / threads));
    for (auto& th : pool) th.join();
}

// ------------------------------------------------ NZ-tiled KV4/FP8 cache (fused decoder's format)
//
// The cache the reference's fused decoder reads (head size 256 only,
// include/turboquant_fused_decode_opt.hpp:10,:85-88):
//   * packed planes: byte `column` (0..127) of (slot, kv head) holds channel `column` in bits
//     3:0 and channel `column + 128` in bits 7:4 (tests/common/fused_decode_opt_fixture.hpp:
//     286-293), at NzTiledPackedByte(slot, head, column, H, 128) inside the page
//     (kernels/ops/turboquant/fused_decode/common/turboquant_layout.h:80-92): 64-row tiles,
//     [tile][kv head][32-byte column group][row][byte];
//   * a nibble is a two's-complement code c in [-8, 7] and stands for (c + 0.5) * scale / gain
//     -- the uniform mid-rise grid b - 7.5 with b = c + 8, gain 2.9832882881
//     (fused_decode/common/turboquant_mode.h:100-124; the decode multiplies the key scale by
//     softmax_scale / gain and the value scale by 1 / gain,
//     fused_decode/vector/turboquant_vector_service.h:592-593,:754-755);
//   * scales: ceil(2H / 8) * 8 floats per slot, key scales of the H heads first, value scales
//     after them (fused_decode/common/turboquant_common.h:62-65; fixture :283-284).
static inline std::size_t nz_tiled_packed_byte(std::size_t slot, std::size_t head, std::size_t column,
                                               std::size_t H, std::size_t packed_bytes)
{
    const std::size_t tile_row = slot % 64;
    return (slot - tile_row) * H * packed_bytes + head * 64 * packed_bytes +
           ((column / 32) * 64 + tile_row) * 32 + column % 32;
}
static inline int s4(unsigned nibble) { return static_cast<int>(nibble ^ 8u) - 8; }

std::size_t tqo_nz_tiled_packed_byte(std::size_t slot, std::size_t head, std::size_t column,
                                     std::size_t H, std::size_t packed_bytes)
{
    return nz_tiled_packed_byte(slot, head, column, H, packed_bytes);
}

// The import this library performs before it decodes such a cache: codes unchanged, re-paired
// into the native planes (key: token-major, channels 2j | 2j+1 per byte; value: channel-major
// inside each 16-token strip, tokens 2j | 2j+1 per byte), scale = FP32 (slot scale / gain),
// planar. Pages keep their numbers. Returns 0, or -1 on a geometry the format does not have.
int tqo_nz_kv4_import(const std::uint8_t* nz_key, const std::uint8_t* nz_value, const float* nz_scales,
                      int H, int S, int P, float gain, std::uint8_t* key_cache,
                      std::uint8_t* value_cache, float* scale_cache)
{
    constexpr int d = 256, packed = 128;
    if (H < 1 || (S != 64 && S != 128) || P < 0) return -1;
    const int slot_floats = (2 * H + 7) / 8 * 8;
    std::vector<int> code(d);
    for (int page = 0; page < P; ++page)
        for (int row = 0; row < S; ++row)
            for (int head = 0; head < H; ++head)
                for (int plane = 0; plane < 2; ++plane) {
                    const std::uint8_t* src = (plane ? nz_value : nz_key) +
                                              static_cast<std::size_t>(page) * S * H * packed;
                    for (int col = 0; col < packed; ++col) {
                        const unsigned b = src[nz_tiled_packed_byte(row, head, col, H, packed)];
                        code[col] = b & 15u;
                        code[col + packed] = b >> 4;
                    }
                    const std::size_t block = (static_cast<std::size_t>(page) * H + head) * S * (d / 2);
                    for (int ch = 0; ch < d; ++ch) {
                        std::size_t nib;
                        if (plane == 0) nib = static_cast<std::size_t>(row) * d + ch;
                        else nib = static_cast<std::size_t>(row / kStrip) * (kStrip * d) + ch * kStrip + row % kStrip;
                        std::uint8_t* dst = (plane ? value_cache : key_cache) + block + nib / 2;
                        const unsigned shift = (nib & 1) ? 4u : 0u;
                        *dst = static_cast<std::uint8_t>((*dst & ~(15u << shift)) | (code[ch] << shift));
                    }
                    const float sc = nz_scales[(static_cast<std::size_t>(page) * S + row) * slot_floats +
                                               plane * H + head];
                    scale_cache[((static_cast<std::size_t>(plane) * P + page) * H + head) * S + row] = sc / gain;
                }
    return 0;
}

// Pi = diag(s) H diag(s) / sqrt(d) of the fused decoder, H the Sylvester-Hadamard matrix
// (tests/common/fused_decode_opt_fixture.hpp:104-117,:166-182: x *= s, the unnormalised
// butterfly, x *= s, one multiply by inv_sqrt_len), on `rows` vectors in FP64, narrowed once.
void tqo_signed_hadamard(int d, const float* signs, const float* x, float* y, int rows)
{
    std::vector<double> v(d);
    double scale = 1.0;
    for (int n = d; n > 1; n >>= 2) scale *= 0.5;   // d is a power of four here (64, 256) or 128
    if (d == 128) scale = 1.0 / std::sqrt(128.0);
    for (int r = 0; r < rows; ++r) {
        for (int i = 0; i < d; ++i) v[i] = static_cast<double>(x[static_cast<std::size_t>(r) * d + i]) * signs[i];
        for (int stride = 1; stride < d; stride <<= 1)
            for (int i = 0; i < d; ++i)
                if ((i & stride) == 0) {
                    const double a = v[i], b = v[i ^ stride];
                    v[i] = a + b;
                    v[i ^ stride] = a - b;
                }
        for (int i = 0; i < d; ++i)
            y[static_cast<std::size_t>(r) * d + i] = static_cast<float>(v[i] * signs[i] * scale);
    }
}

// FP64 attention straight off the NZ-tiled cache with a pre-rotated FP32 query
// [B][Hq][256] (the fused decoder's `queryRot`), output in the rotated basis, FP32
// (the scalar FP64 sum of tests/common/fused_decode_opt_fixture.hpp:300-312, for arbitrary
// cache contents). Scales enter as the FP32 quotient scale / gain, as in the import above.
// `levels` (16 floats, or null): the value a stored nibble stands for. Null is the uniform
// mid-rise grid (nibble n as a signed 4-bit number + 0.5); the fused decoder's Lloyd-Max toggle
// keeps the storage (bin b stored as the signed nibble b - 8) and reconstructs levels[b]
// (kernels/ops/turboquant/fused_decode/common/turboquant_codec_mx.h:61-72), gain 1.
static void nz_kv4_decode_levels(const float* q_rot, const std::uint8_t* nz_key, const std::uint8_t* nz_value,
                                 const float* nz_scales, const std::int32_t* block_tables,
                                 const std::int32_t* context_lens, int B, int Hq, int H, int S, int max_blocks,
                                 float softmax_scale, float gain, const float* levels, float* out);

void tqo_nz_kv4_decode(const float* q_rot, const std::uint8_t* nz_key, const std::uint8_t* nz_value,
                       const float* nz_scales, const std::int32_t* block_tables,
                       const std::int32_t* context_lens, int B, int Hq, int H, int S, int max_blocks,
                       float softmax_scale, float gain, float* out)
{
    nz_kv4_decode_levels(q_rot, nz_key, nz_value, nz_scales, block_tables, context_lens, B, Hq, H, S, max_blocks,
                         softmax_scale, gain, nullptr, out);
}

// The e4m3-rounded 16-level Lloyd-Max table of the fused decoder's KV4/FP8 mode
// (kernels/ops/turboquant/fused_decode/common/turboquant_mode.h:191-197): Max's table for
// N(0,1), each entry rounded to the nearest fp8 e4m3 value; odd, ascending with the bin index.
void tqo_kv4_lloydmax_lut(float* levels16)
{
    static const float half[8] = {0.125f, 0.375f, 0.6875f, 0.9375f, 1.25f, 1.625f, 2.0f, 2.75f};
    for (int i = 0; i < 8; ++i) {
        levels16[8 + i] = half[i];
        levels16[7 - i] = -half[i];
    }
}

// The same decode over a cache written on the Lloyd-Max codebook: levels by bin index, gain 1.
void tqo_nz_kv4_decode_lut(const float* q_rot, const std::uint8_t* nz_key, const std::uint8_t* nz_value,
                           const float* nz_scales, const std::int32_t* block_tables,
                           const std::int32_t* context_lens, int B, int Hq, int H, int S, int max_blocks,
                           float softmax_scale, const float* levels16, float* out)
{
    nz_kv4_decode_levels(q_rot, nz_key, nz_value, nz_scales, block_tables, context_lens, B, Hq, H, S, max_blocks,
                         softmax_scale, 1.0f, levels16, out);
}

static void nz_kv4_decode_levels(const float* q_rot, const std::uint8_t* nz_key, const std::uint8_t* nz_value,
                                 const float* nz_scales, const std::int32_t* block_tables,
                                 const std::int32_t* context_lens, int B, int Hq, int H, int S, int max_blocks,
                                 float softmax_scale, float gain, const float* levels, float* out)
{
    constexpr int d = 256, packed = 128;
    // nibble n -> its value: the signed nibble + 0.5, or the level of bin b = n ^ 8 (n is b - 8 in four bits)
    auto value_of = [&](unsigned n) {
        return levels ? static_cast<double>(levels[(n ^ 8u) & 15u]) : s4(n) + 0.5;
    };
    const int G = Hq / H, slot_floats = (2 * H + 7) / 8 * 8;
    for (int b = 0; b < B; ++b)
        for (int qh = 0; qh < Hq; ++qh) {
            const int head = qh / G, ctx = std::max(0, context_lens[b]);
            const float* q = q_rot + (static_cast<std::size_t>(b) * Hq + qh) * d;
            float* o = out + (static_cast<std::size_t>(b) * Hq + qh) * d;
            std::vector<double> score(ctx), acc(d, 0.0);
            double m = -std::numeric_limits<double>::infinity();
            auto plane_base = [&](const std::uint8_t* pool, int t) {
                const std::size_t page = static_cast<std::size_t>(block_tables[b * max_blocks + t / S]);
                return pool + page * S * H * packed;
            };
            auto scale_of = [&](int t, int plane) {
                const std::size_t page = static_cast<std::size_t>(block_tables[b * max_blocks + t / S]);
                return static_cast<double>(nz_scales[(page * S + t % S) * slot_floats + plane * H + head] / gain);
            };
            for (int t = 0; t < ctx; ++t) {
                const std::uint8_t* kp = plane_base(nz_key, t);
                double dot = 0.0;
                for (int col = 0; col < packed; ++col) {
                    const unsigned byte = kp[nz_tiled_packed_byte(t % S, head, col, H, packed)];
                    dot += static_cast<double>(q[col]) * value_of(byte & 15u) +
                           static_cast<double>(q[col + packed]) * value_of(byte >> 4);
                }
                score[t] = dot * scale_of(t, 0) * static_cast<double>(softmax_scale);
                m = std::max(m, score[t]);
            }
            double l = 0.0;
            for (int t = 0; t < ctx; ++t) {
                const double p = std::exp(score[t] - m), vs = scale_of(t, 1);
                l += p;
                const std::uint8_t* vp = plane_base(nz_value, t);
                for (int col = 0; col < packed; ++col) {
                    const unsigned byte = vp[nz_tiled_packed_byte(t % S, head, col, H, packed)];
                    acc[col] += p * vs * value_of(byte & 15u);
                    acc[col + packed] += p * vs * value_of(byte >> 4);
                }
            }
            for (int c = 0; c < d; ++c) o[c] = ctx > 0 ? static_cast<float>(acc[c] / l) : 0.0f;
        }
}

int tqo_hardware_threads() { return static_cast<int>(std::thread::hardware_concurrency()); }

}  // extern "C"
