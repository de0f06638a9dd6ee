// GGUF v3 container reader / writer and host codecs for the ggml block formats this engine
// loads: F32, F16, BF16, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K (256-element super-blocks with packed
// 6-bit sub-scales) and MXFP4.  The reader memory-maps the file; tensors are exposed by index
// or name with their raw bytes, and any supported type can be dequantised to fp32.  Quantisers
// exist for Q8_0, Q4_K and Q6_K so that random-init checkpoints can be written in valid GGUF.
//
// Reference components: GgufReader (src/model/weight_loader/gguf_reader.cpp), block specs
// src/model/quantization/gguf_kquant.h:49-57 (Q2_K 84 B/256, Q3_K 110, Q4_K 144, Q5_K 176,
// Q6_K 210, Q8_0 34 B/32, MXFP4 17 B/32) and the MXFP4 host dequantiser.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "lsb_runtime.h"

namespace lsb {

enum GgmlType { T_F32 = 0, T_F16 = 1, T_Q8_0 = 8, T_Q2_K = 10, T_Q3_K = 11, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_I32 = 26, T_BF16 = 30, T_MXFP4 = 39 };

static inline float h2f(uint16_t h) {
    const uint32_t s = (h & 0x8000u) << 16, e = (h >> 10) & 0x1f, m = h & 0x3ff;
    uint32_t u;
    if (e == 0) {
        if (m == 0) u = s;
        else {
            int ee = -1;
            uint32_t mm = m;
            do { ++ee; mm <<= 1; } while (!(mm & 0x400));
            u = s | ((uint32_t)(127 - 15 - ee) << 23) | ((mm & 0x3ff) << 13);
        }
    } else if (e == 31) u = s | 0x7f800000u | (m << 13);
    else u = s | ((e + 112) << 23) | (m << 13);
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
static inline uint16_t f2h(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t s = (x >> 16) & 0x8000u;
    int e = (int)((x >> 23) & 0xff) - 127 + 15;
    uint32_t m = x & 0x7fffffu;
    if (((x >> 23) & 0xff) == 0xff) return (uint16_t)(s | 0x7c00u | (m ? 0x200u : 0));
    if (e >= 31) return (uint16_t)(s | 0x7c00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)s;
        m |= 0x800000u;
        const int shift = 14 - e;
        uint32_t r = m >> shift;
        const uint32_t rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (r & 1))) ++r;
        return (uint16_t)(s | r);
    }
    uint32_t r = (uint32_t)(e << 10) | (m >> 13);
    const uint32_t rem = m & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) ++r;
    return (uint16_t)(s | r);
}

int type_block_elems(int t) {
    switch (t) {
        case T_F32: case T_F16: case T_BF16: case T_I32: return 1;
        case T_Q8_0: case T_MXFP4: return 32;
        case T_Q2_K: case T_Q3_K: case T_Q4_K: case T_Q5_K: case T_Q6_K: return 256;
        default: return 0;
    }
}
int type_block_bytes(int t) {
    switch (t) {
        case T_F32: case T_I32: return 4;
        case T_F16: case T_BF16: return 2;
        case T_Q8_0: return 34;
        case T_MXFP4: return 17;
        case T_Q2_K: return 84;
        case T_Q3_K: return 110;
        case T_Q4_K: return 144;
        case T_Q5_K: return 176;
        case T_Q6_K: return 210;
        default: return 0;
    }
}

static inline void scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
    if (j < 4) { *d = q[j] & 63; *m = q[j + 4] & 63; }
    else { *d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

static const float kFp4[16] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -0.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

int dequantize(int type, const uint8_t* src, float* y, int64_t n) {
    const int be = type_block_elems(type), bb = type_block_bytes(type);
    if (!be || n % be) return LSB_ERR_FORMAT;
    const int64_t nb = n / be;
    switch (type) {
        case T_F32: std::memcpy(y, src, n * 4); return 0;
        case T_I32: for (int64_t i = 0; i < n; ++i) { int32_t v; std::memcpy(&v, src + 4 * i, 4); y[i] = (float)v; } return 0;   // integer tables (exact below 2^24)
        case T_F16: for (int64_t i = 0; i < n; ++i) { uint16_t h; std::memcpy(&h, src + 2 * i, 2); y[i] = h2f(h); } return 0;
        case T_BF16: for (int64_t i = 0; i < n; ++i) { uint16_t h; std::memcpy(&h, src + 2 * i, 2); uint32_t u = (uint32_t)h << 16; std::memcpy(&y[i], &u, 4); } return 0;
        case T_Q8_0:
            for (int64_t b = 0; b < nb; ++b) {
                const uint8_t* p = src + b * bb; uint16_t dh; std::memcpy(&dh, p, 2); const float d = h2f(dh);
                const int8_t* q = (const int8_t*)(p + 2);
                for (int i = 0; i < 32; ++i) y[b * 32 + i] = d * q[i];
            }
            return 0;
        case T_MXFP4:
            for (int64_t b = 0; b < nb; ++b) {
                const uint8_t* p = src + b * bb;
                const float d = std::ldexp(1.0f, (int)p[0] - 127);
                for (int i = 0; i < 16; ++i) { y[b * 32 + i] = kFp4[p[1 + i] & 0xF] * d; y[b * 32 + 16 + i] = kFp4[p[1 + i] >> 4] * d; }
            }
            return 0;
        case T_Q4_K:
            for (int64_t b = 0; b < nb; ++b) {
                const uint8_t* p = src + b * bb; uint16_t dh, mh; std::memcpy(&dh, p, 2); std::memcpy(&mh, p + 2, 2);
                const float d = h2f(dh), dmin = h2f(mh);
                const uint8_t* sc = p + 4; const uint8_t* q = p + 16; float* o = y + b * 256; int is = 0;
                for (int j = 0; j < 256; j += 64) {
                    uint8_t s1, m1, s2, m2; scale_min_k4(is, sc, &s1, &m1); scale_min_k4(is + 1, sc, &s2, &m2);
                    for (int l = 0; l < 32; ++l) o[j + l] = d * s1 * (q[l] & 0xF) - dmin * m1;
                    for (int l = 0; l < 32; ++l) o[j + 32 + l] = d * s2 * (q[l] >> 4) - dmin * m2;
                    q += 32; is += 2;
                }
            }
            return 0;
        case T_Q5_K:
            for (int64_t b = 0; b < nb; ++b) {
                const uint8_t* p = src + b * bb; uint16_t dh, mh; std::memcpy(&dh, p, 2); std::memcpy(&mh, p + 2, 2);
                const float d = h2f(dh), dmin = h2f(mh);
                const uint8_t* sc = p + 4; const uint8_t* qh = p + 16; const uint8_t* ql = p + 48; float* o = y + b * 256;
                int is = 0; uint8_t u1 = 1, u2 = 2;
                for (int j = 0; j < 256; j += 64) {
                    uint8_t s1, m1, s2, m2; scale_min_k4(is, sc, &s1, &m1); scale_min_k4(is + 1, sc, &s2, &m2);
                    for (int l = 0; l < 32; ++l) o[j + l] = d * s1 * ((ql[l] & 0xF) + ((qh[l] & u1) ? 16 : 0)) - dmin * m1;
                    for (int l = 0; l < 32; ++l) o[j + 32 + l] = d * s2 * ((ql[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - dmin * m2;
                    ql += 32; is += 2; u1 <<= 2; u2 <<= 2;
                }
            }
            return 0;
        case T_Q6_K:
            for (int64_t b = 0; b < nb; ++b) {
                const uint8_t* p = src + b * bb; const uint8_t* ql = p; const uint8_t* qh = p + 128; const int8_t* sc = (const int8_t*)(p + 192);
                uint16_t dh; std::memcpy(&dh, p + 208, 2); const float d = h2f(dh); float* o = y + b * 256;
                for (int n2 = 0; n2 < 256; n2 += 128) {
                    for (int l = 0; l < 32; ++l) {
                        const int is = l / 16;
                        const int q1 = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                        const int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                        const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                        const int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                        o[l] = d * sc[is + 0] * q1; o[l + 32] = d * sc[is + 2] * q2; o[l + 64] = d * sc[is + 4] * q3; o[l + 96] = d * sc[is + 6] * q4;
                    }
                    o += 128; ql += 64; qh += 32; sc += 8;
                }
            }
            return 0;
        case T_Q2_K:
            for (int64_t b = 0; b < nb; ++b) {
                const uint8_t* p = src + b * bb; const uint8_t* sc = p; const uint8_t* q = p + 16;
                uint16_t dh, mh; std::memcpy(&dh, p + 80, 2); std::memcpy(&mh, p + 82, 2);
                const float d = h2f(dh), dmin = h2f(mh); float* o = y + b * 256; int is = 0;
                for (int n2 = 0; n2 < 256; n2 += 128) {
                    int shift = 0;
                    for (int j = 0; j < 4; ++j) {
                        uint8_t s = sc[is++]; float dl = d * (s & 0xF), ml = dmin * (s >> 4);
                        for (int l = 0; l < 16; ++l) *o++ = dl * ((q[l] >> shift) & 3) - ml;
                        s = sc[is++]; dl = d * (s & 0xF); ml = dmin * (s >> 4);
                        for (int l = 0; l < 16; ++l) *o++ = dl * ((q[l + 16] >> shift) & 3) - ml;
                        shift += 2;
                    }
                    q += 32;
                }
            }
            return 0;
        case T_Q3_K:
            for (int64_t b = 0; b < nb; ++b) {
                const uint8_t* p = src + b * bb; const uint8_t* hm = p; const uint8_t* q = p + 32; const uint8_t* s12 = p + 96;
                uint16_t dh; std::memcpy(&dh, p + 108, 2); const float d_all = h2f(dh);
                uint32_t aux[4]; std::memcpy(aux, s12, 12);
                const uint32_t kmask1 = 0x03030303, kmask2 = 0x0f0f0f0f; const uint32_t tmp = aux[2];
                aux[2] = ((aux[0] >> 4) & kmask2) | (((tmp >> 4) & kmask1) << 4);
                aux[3] = ((aux[1] >> 4) & kmask2) | (((tmp >> 6) & kmask1) << 4);
                aux[0] = (aux[0] & kmask2) | (((tmp >> 0) & kmask1) << 4);
                aux[1] = (aux[1] & kmask2) | (((tmp >> 2) & kmask1) << 4);
                const int8_t* scales = (const int8_t*)aux; float* o = y + b * 256; int is = 0; uint8_t m = 1;
                for (int n2 = 0; n2 < 256; n2 += 128) {
                    int shift = 0;
                    for (int j = 0; j < 4; ++j) {
                        float dl = d_all * (scales[is++] - 32);
                        for (int l = 0; l < 16; ++l) *o++ = dl * ((int8_t)((q[l] >> shift) & 3) - ((hm[l] & m) ? 0 : 4));
                        dl = d_all * (scales[is++] - 32);
                        for (int l = 0; l < 16; ++l) *o++ = dl * ((int8_t)((q[l + 16] >> shift) & 3) - ((hm[l + 16] & m) ? 0 : 4));
                        shift += 2; m <<= 1;
                    }
                    q += 32;
                }
            }
            return 0;
        default: return LSB_ERR_FORMAT;
    }
}

// ---- quantisers (round-trip quality, not bit-compatible with any particular encoder) -----------
static void quant_q8_0(const float* x, uint8_t* dst, int64_t n) {
    for (int64_t b = 0; b < n / 32; ++b) {
        float amax = 0; for (int i = 0; i < 32; ++i) amax = std::max(amax, std::fabs(x[b * 32 + i]));
        const float d = amax / 127.f, id = d ? 1.f / d : 0.f;
        const uint16_t dh = f2h(d); std::memcpy(dst + b * 34, &dh, 2);
        for (int i = 0; i < 32; ++i) ((int8_t*)(dst + b * 34 + 2))[i] = (int8_t)std::lround(x[b * 32 + i] * id);
    }
}
static void quant_q4_k(const float* x, uint8_t* dst, int64_t n) {
    for (int64_t b = 0; b < n / 256; ++b) {
        const float* xb = x + b * 256; uint8_t* p = dst + b * 144;
        float sc[8], mn[8]; float max_sc = 0, max_mn = 0;
        for (int j = 0; j < 8; ++j) {
            float lo = xb[j * 32], hi = xb[j * 32];
            for (int i = 1; i < 32; ++i) { lo = std::min(lo, xb[j * 32 + i]); hi = std::max(hi, xb[j * 32 + i]); }
            if (lo > 0) lo = 0;
            sc[j] = (hi - lo) / 15.f; mn[j] = -lo;
            max_sc = std::max(max_sc, sc[j]); max_mn = std::max(max_mn, mn[j]);
        }
        const float d = max_sc / 63.f, dmin = max_mn / 63.f;
        const uint16_t dh = f2h(d), mh = f2h(dmin); std::memcpy(p, &dh, 2); std::memcpy(p + 2, &mh, 2);
        const float dq = h2f(dh), dminq = h2f(mh);
        uint8_t ls[8], lm[8];
        for (int j = 0; j < 8; ++j) { ls[j] = (uint8_t)std::min(63L, std::lround(dq ? sc[j] / dq : 0)); lm[j] = (uint8_t)std::min(63L, std::lround(dminq ? mn[j] / dminq : 0)); }
        uint8_t* s = p + 4; std::memset(s, 0, 12);
        for (int j = 0; j < 8; ++j) {
            if (j < 4) { s[j] = ls[j]; s[j + 4] = lm[j]; }
            else { s[j + 4] = (ls[j] & 0xF) | ((lm[j] & 0xF) << 4); s[j - 4] |= (ls[j] >> 4) << 6; s[j] |= (lm[j] >> 4) << 6; }
        }
        uint8_t* q = p + 16;
        for (int j = 0; j < 8; j += 2) {
            for (int l = 0; l < 32; ++l) {
                int v[2];
                for (int h = 0; h < 2; ++h) {
                    const float dd = dq * ls[j + h], mm = dminq * lm[j + h];
                    v[h] = dd ? (int)std::lround((xb[(j + h) * 32 + l] + mm) / dd) : 0;
                    v[h] = std::max(0, std::min(15, v[h]));
                }
                q[l] = (uint8_t)(v[0] | (v[1] << 4));
            }
            q += 32;
        }
    }
}
static void quant_q6_k(const float* x, uint8_t* dst, int64_t n) {
    for (int64_t b = 0; b < n / 256; ++b) {
        const float* xb = x + b * 256; uint8_t* p = dst + b * 210;
        float scl[16]; float maxs = 0;
        for (int j = 0; j < 16; ++j) { float am = 0; for (int i = 0; i < 16; ++i) am = std::max(am, std::fabs(xb[j * 16 + i])); scl[j] = am / 31.f; maxs = std::max(maxs, scl[j]); }
        const float d = maxs / 127.f; const uint16_t dh = f2h(d); const float dq = h2f(dh); std::memcpy(p + 208, &dh, 2);
        int8_t* sc = (int8_t*)(p + 192); int L[256];
        for (int j = 0; j < 16; ++j) {
            sc[j] = (int8_t)std::min(127L, std::lround(dq ? scl[j] / dq : 0));
            const float dd = dq * sc[j];
            for (int i = 0; i < 16; ++i) { int v = dd ? (int)std::lround(xb[j * 16 + i] / dd) : 0; L[j * 16 + i] = std::max(-32, std::min(31, v)) + 32; }
        }
        uint8_t* ql = p; uint8_t* qh = p + 128;
        for (int n2 = 0; n2 < 256; n2 += 128) {
            for (int l = 0; l < 32; ++l) {
                const int q1 = L[n2 + l], q2 = L[n2 + l + 32], q3 = L[n2 + l + 64], q4 = L[n2 + l + 96];
                ql[l] = (uint8_t)((q1 & 0xF) | ((q3 & 0xF) << 4)); ql[l + 32] = (uint8_t)((q2 & 0xF) | ((q4 & 0xF) << 4));
                qh[l] = (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
            }
            ql += 64; qh += 32;
        }
    }
}
int quantize(int type, const float* x, uint8_t* dst, int64_t n) {
    const int be = type_block_elems(type);
    if (!be || n % be) return LSB_ERR_FORMAT;
    switch (type) {
        case T_F32: std::memcpy(dst, x, n * 4); return 0;
        case T_F16: for (int64_t i = 0; i < n; ++i) { uint16_t h = f2h(x[i]); std::memcpy(dst + 2 * i, &h, 2); } return 0;
        case T_BF16: for (int64_t i = 0; i < n; ++i) { uint32_t u; std::memcpy(&u, &x[i], 4); u += 0x7fffu + ((u >> 16) & 1); uint16_t h = (uint16_t)(u >> 16); std::memcpy(dst + 2 * i, &h, 2); } return 0;
        case T_Q8_0: quant_q8_0(x, dst, n); return 0;
        case T_Q4_K: quant_q4_k(x, dst, n); return 0;
        case T_Q6_K: quant_q6_k(x, dst, n); return 0;
        default: return LSB_ERR_FORMAT;
    }
}

// ---- container -------------------------------------------------------------------------------
struct MetaVal { int type = -1; uint64_t u = 0; double f = 0; std::string s; int arr_type = -1; std::vector<std::string> arr_s; std::vector<double> arr_n; };
struct TensorInfo { std::string name; int type = 0; int ndims = 0; uint64_t dims[4] = {1, 1, 1, 1}; uint64_t offset = 0; uint64_t nbytes = 0; };

class GgufFile {
public:
    ~GgufFile() { if (base_) munmap((void*)base_, size_); if (fd_ >= 0) close(fd_); }
    int open(const char* path) {
        fd_ = ::open(path, O_RDONLY);
        if (fd_ < 0) return LSB_ERR_IO;
        struct stat st; if (fstat(fd_, &st)) return LSB_ERR_IO;
        size_ = (size_t)st.st_size;
        base_ = (const uint8_t*)mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
        if (base_ == MAP_FAILED) { base_ = nullptr; return LSB_ERR_IO; }
        return parse();
    }
    std::map<std::string, MetaVal> meta;
    std::vector<TensorInfo> tensors;
    std::map<std::string, int> index;
    const uint8_t* data() const { return base_ + data_off_; }
    int version = 0;

private:
    bool rd(void* dst, size_t n) { if (pos_ + n > size_) return false; std::memcpy(dst, base_ + pos_, n); pos_ += n; return true; }
    bool rd_str(std::string* s) { uint64_t n; if (!rd(&n, 8) || pos_ + n > size_) return false; s->assign((const char*)base_ + pos_, n); pos_ += n; return true; }
    bool rd_scalar(int t, MetaVal* v) {
        switch (t) {
            case 0: { uint8_t x; if (!rd(&x, 1)) return false; v->u = x; v->f = x; return true; }
            case 1: { int8_t x; if (!rd(&x, 1)) return false; v->u = (uint64_t)(int64_t)x; v->f = x; return true; }
            case 2: { uint16_t x; if (!rd(&x, 2)) return false; v->u = x; v->f = x; return true; }
            case 3: { int16_t x; if (!rd(&x, 2)) return false; v->u = (uint64_t)(int64_t)x; v->f = x; return true; }
            case 4: { uint32_t x; if (!rd(&x, 4)) return false; v->u = x; v->f = x; return true; }
            case 5: { int32_t x; if (!rd(&x, 4)) return false; v->u = (uint64_t)(int64_t)x; v->f = x; return true; }
            case 6: { float x; if (!rd(&x, 4)) return false; v->f = x; v->u = (uint64_t)x; return true; }
            case 7: { uint8_t x; if (!rd(&x, 1)) return false; v->u = x; v->f = x; return true; }
            case 8: return rd_str(&v->s);
            case 10: { uint64_t x; if (!rd(&x, 8)) return false; v->u = x; v->f = (double)x; return true; }
            case 11: { int64_t x; if (!rd(&x, 8)) return false; v->u = (uint64_t)x; v->f = (double)x; return true; }
            case 12: { double x; if (!rd(&x, 8)) return false; v->f = x; v->u = (uint64_t)x; return true; }
            default: return false;
        }
    }
    int parse() {
        uint32_t magic; uint64_t nt, nkv; uint32_t ver;
        if (!rd(&magic, 4) || magic != 0x46554747u) return LSB_ERR_FORMAT;
        if (!rd(&ver, 4) || ver < 2 || ver > 3) return LSB_ERR_FORMAT;
        version = (int)ver;
        if (!rd(&nt, 8) || !rd(&nkv, 8)) return LSB_ERR_FORMAT;
        for (uint64_t i = 0; i < nkv; ++i) {
            std::string key; uint32_t t; if (!rd_str(&key) || !rd(&t, 4)) return LSB_ERR_FORMAT;
            MetaVal v; v.type = (int)t;
            if (t == 9) {
                uint32_t at; uint64_t cnt; if (!rd(&at, 4) || !rd(&cnt, 8)) return LSB_ERR_FORMAT;
                v.arr_type = (int)at;
                for (uint64_t j = 0; j < cnt; ++j) {
                    MetaVal e; if (!rd_scalar((int)at, &e)) return LSB_ERR_FORMAT;
                    if (at == 8) v.arr_s.push_back(std::move(e.s)); else v.arr_n.push_back(e.f);
                }
            } else if (!rd_scalar((int)t, &v)) return LSB_ERR_FORMAT;
            meta[key] = std::move(v);
        }
        uint64_t align = 32;
        auto it = meta.find("general.alignment"); if (it != meta.end() && it->second.u) align = it->second.u;
        for (uint64_t i = 0; i < nt; ++i) {
            TensorInfo ti; uint32_t nd, ty;
            if (!rd_str(&ti.name) || !rd(&nd, 4) || nd > 4) return LSB_ERR_FORMAT;
            ti.ndims = (int)nd;
            for (uint32_t d = 0; d < nd; ++d) if (!rd(&ti.dims[d], 8)) return LSB_ERR_FORMAT;
            if (!rd(&ty, 4) || !rd(&ti.offset, 8)) return LSB_ERR_FORMAT;
            ti.type = (int)ty;
            uint64_t ne = 1; for (uint32_t d = 0; d < nd; ++d) ne *= ti.dims[d];
            const int be = type_block_elems(ti.type), bb = type_block_bytes(ti.type);
            ti.nbytes = be ? ne / be * bb : 0;
            index[ti.name] = (int)tensors.size();
            tensors.push_back(std::move(ti));
        }
        data_off_ = (pos_ + align - 1) / align * align;
        for (auto& t : tensors) if (data_off_ + t.offset + t.nbytes > size_) return LSB_ERR_FORMAT;
        return 0;
    }
    int fd_ = -1; const uint8_t* base_ = nullptr; size_t size_ = 0, pos_ = 0, data_off_ = 0;
};

class GgufWriter {
public:
    void meta_u32(const std::string& k, uint32_t v) { put_str(kv_, k); put(kv_, (uint32_t)4); put(kv_, v); ++nkv_; }
    void meta_f32(const std::string& k, float v) { put_str(kv_, k); put(kv_, (uint32_t)6); put(kv_, v); ++nkv_; }
    void meta_str(const std::string& k, const std::string& v) { put_str(kv_, k); put(kv_, (uint32_t)8); put_str(kv_, v); ++nkv_; }
    void meta_str_array(const std::string& k, const std::vector<std::string>& v) {
        put_str(kv_, k); put(kv_, (uint32_t)9); put(kv_, (uint32_t)8); put(kv_, (uint64_t)v.size());
        for (auto& s : v) put_str(kv_, s);
        ++nkv_;
    }
    void meta_i32_array(const std::string& k, const int32_t* v, uint64_t n) {
        put_str(kv_, k); put(kv_, (uint32_t)9); put(kv_, (uint32_t)5); put(kv_, n);
        for (uint64_t i = 0; i < n; ++i) put(kv_, v[i]);
        ++nkv_;
    }
    int add_tensor(const std::string& name, int type, int ndims, const uint64_t* dims, const void* data, uint64_t nbytes) {
        TensorInfo t; t.name = name; t.type = type; t.ndims = ndims;
        for (int i = 0; i < ndims; ++i) t.dims[i] = dims[i];
        t.offset = (blob_.size() + 31) / 32 * 32;
        blob_.resize(t.offset + nbytes);
        std::memcpy(blob_.data() + t.offset, data, nbytes);
        t.nbytes = nbytes; infos_.push_back(t);
        return 0;
    }
    int finish(const char* path) {
        std::vector<uint8_t> h;
        put(h, (uint32_t)0x46554747u); put(h, (uint32_t)3); put(h, (uint64_t)infos_.size()); put(h, (uint64_t)nkv_);
        h.insert(h.end(), kv_.begin(), kv_.end());
        for (auto& t : infos_) {
            put_str(h, t.name); put(h, (uint32_t)t.ndims);
            for (int i = 0; i < t.ndims; ++i) put(h, (uint64_t)t.dims[i]);
            put(h, (uint32_t)t.type); put(h, (uint64_t)t.offset);
        }
        h.resize((h.size() + 31) / 32 * 32);
        FILE* f = std::fopen(path, "wb");
        if (!f) return LSB_ERR_IO;
        bool ok = std::fwrite(h.data(), 1, h.size(), f) == h.size() && std::fwrite(blob_.data(), 1, blob_.size(), f) == blob_.size();
        std::fclose(f);
        return ok ? 0 : LSB_ERR_IO;
    }
private:
    template <class T> static void put(std::vector<uint8_t>& b, T v) { const uint8_t* p = (const uint8_t*)&v; b.insert(b.end(), p, p + sizeof(T)); }
    static void put_str(std::vector<uint8_t>& b, const std::string& s) { put(b, (uint64_t)s.size()); b.insert(b.end(), s.begin(), s.end()); }
    std::vector<uint8_t> kv_, blob_; std::vector<TensorInfo> infos_; uint64_t nkv_ = 0;
};

}  // namespace lsb

using namespace lsb;
extern "C" {
LSB_RT_API int lsb_ggml_block_elems(int type) { return type_block_elems(type); }
LSB_RT_API int lsb_ggml_block_bytes(int type) { return type_block_bytes(type); }
LSB_RT_API int lsb_ggml_dequantize(int type, const void* src, float* dst, long long n) { return dequantize(type, (const uint8_t*)src, dst, n); }
LSB_RT_API int lsb_ggml_quantize(int type, const float* src, void* dst, long long n) { return quantize(type, src, (uint8_t*)dst, n); }

LSB_RT_API void* lsb_gguf_open(const char* path, int* rc) {
    auto* g = new GgufFile();
    int r = g->open(path);
    if (rc) *rc = r;
    if (r) { delete g; return nullptr; }
    return g;
}
LSB_RT_API void lsb_gguf_close(void* h) { delete (GgufFile*)h; }
LSB_RT_API int lsb_gguf_version(void* h) { return ((GgufFile*)h)->version; }
LSB_RT_API int lsb_gguf_n_tensors(void* h) { return (int)((GgufFile*)h)->tensors.size(); }
LSB_RT_API int lsb_gguf_find(void* h, const char* name) { auto& ix = ((GgufFile*)h)->index; auto it = ix.find(name); return it == ix.end() ? -1 : it->second; }
LSB_RT_API int lsb_gguf_tensor_info(void* h, int i, char* name, int cap, int* type, int* ndims, unsigned long long* dims, unsigned long long* nbytes) {
    auto* g = (GgufFile*)h;
    if (i < 0 || i >= (int)g->tensors.size()) return LSB_ERR_ARG;
    const auto& t = g->tensors[i];
    std::snprintf(name, cap, "%s", t.name.c_str());
    *type = t.type; *ndims = t.ndims; for (int d = 0; d < 4; ++d) dims[d] = t.dims[d]; *nbytes = t.nbytes;
    return 0;
}
LSB_RT_API const void* lsb_gguf_tensor_data(void* h, int i) { auto* g = (GgufFile*)h; return g->data() + g->tensors[i].offset; }
LSB_RT_API int lsb_gguf_meta_type(void* h, const char* key) { auto& m = ((GgufFile*)h)->meta; auto it = m.find(key); return it == m.end() ? -1 : it->second.type; }
LSB_RT_API double lsb_gguf_meta_num(void* h, const char* key) { auto& m = ((GgufFile*)h)->meta; auto it = m.find(key); return it == m.end() ? 0.0 : it->second.f; }
LSB_RT_API int lsb_gguf_meta_str(void* h, const char* key, char* out, int cap) {
    auto& m = ((GgufFile*)h)->meta; auto it = m.find(key);
    if (it == m.end()) return -1;
    std::snprintf(out, cap, "%s", it->second.s.c_str());
    return (int)it->second.s.size();
}
LSB_RT_API int lsb_gguf_meta_arr_len(void* h, const char* key) {
    auto& m = ((GgufFile*)h)->meta; auto it = m.find(key);
    if (it == m.end() || it->second.type != 9) return -1;
    return (int)(it->second.arr_type == 8 ? it->second.arr_s.size() : it->second.arr_n.size());
}
LSB_RT_API int lsb_gguf_meta_arr_str(void* h, const char* key, int i, char* out, int cap) {
    auto& m = ((GgufFile*)h)->meta; auto it = m.find(key);
    if (it == m.end() || i < 0 || i >= (int)it->second.arr_s.size()) return -1;
    std::snprintf(out, cap, "%s", it->second.arr_s[i].c_str());
    return (int)it->second.arr_s[i].size();
}
LSB_RT_API double lsb_gguf_meta_arr_num(void* h, const char* key, int i) {
    auto& m = ((GgufFile*)h)->meta; auto it = m.find(key);
    if (it == m.end() || i < 0 || i >= (int)it->second.arr_n.size()) return 0.0;
    return it->second.arr_n[i];
}
LSB_RT_API int lsb_gguf_n_meta(void* h) { return (int)((GgufFile*)h)->meta.size(); }
LSB_RT_API int lsb_gguf_meta_key(void* h, int i, char* out, int cap) {
    auto& m = ((GgufFile*)h)->meta; if (i < 0 || i >= (int)m.size()) return -1;
    auto it = m.begin(); std::advance(it, i);
    std::snprintf(out, cap, "%s", it->first.c_str());
    return (int)it->first.size();
}

LSB_RT_API void* lsb_gguf_writer_new() { return new GgufWriter(); }
LSB_RT_API void lsb_gguf_writer_free(void* w) { delete (GgufWriter*)w; }
LSB_RT_API void lsb_gguf_writer_meta_u32(void* w, const char* k, unsigned int v) { ((GgufWriter*)w)->meta_u32(k, v); }
LSB_RT_API void lsb_gguf_writer_meta_f32(void* w, const char* k, float v) { ((GgufWriter*)w)->meta_f32(k, v); }
LSB_RT_API void lsb_gguf_writer_meta_str(void* w, const char* k, const char* v) { ((GgufWriter*)w)->meta_str(k, v); }
LSB_RT_API void lsb_gguf_writer_meta_str_array(void* w, const char* k, const char* const* items, unsigned long long n) {
    std::vector<std::string> v;
    v.reserve(n);
    for (unsigned long long i = 0; i < n; ++i) v.emplace_back(items[i]);
    ((GgufWriter*)w)->meta_str_array(k, v);
}
LSB_RT_API void lsb_gguf_writer_meta_i32_array(void* w, const char* k, const int* items, unsigned long long n) {
    ((GgufWriter*)w)->meta_i32_array(k, (const int32_t*)items, n);
}
LSB_RT_API int lsb_gguf_writer_add_tensor(void* w, const char* name, int type, int ndims, const unsigned long long* dims, const void* data, unsigned long long nbytes) {
    uint64_t d[4] = {1, 1, 1, 1}; for (int i = 0; i < ndims && i < 4; ++i) d[i] = dims[i];
    return ((GgufWriter*)w)->add_tensor(name, type, ndims, d, data, nbytes);
}
LSB_RT_API int lsb_gguf_writer_finish(void* w, const char* path) { return ((GgufWriter*)w)->finish(path); }
}
