// Host-side checks of the C ABI under AddressSanitizer + UndefinedBehaviorSanitizer (no GPU needed).
//
// What runs: the multi-threaded row packer and the byte-sync helper against plain reference loops, and a
// fuzz of the descriptor validator / plan builder (the code that decides, on the host, what the block kernel
// will be allowed to touch): random and adversarial descriptors -- offsets at and just past every bound,
// negative and enormous values, every kind, both flags -- through sh_block_register and sh_dequant_block_async.
// Every call must come back with a status (never crash, never read or write out of bounds, never overflow
// a signed integer); a descriptor set that is accepted must lie inside the image and the slab.
// On a machine without a CUDA device the calls that get past validation fail in the CUDA runtime and report
// SH_ERR_CUDA, which is fine here: the validator has run by then.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>

#include "../../include/stagehand_b200.h"

static int failures = 0;
#define EXPECT(cond, ...)                          \
    do {                                           \
        if (!(cond)) {                             \
            ++failures;                            \
            fprintf(stderr, "FAILED %s:%d: ", __FILE__, __LINE__); \
            fprintf(stderr, __VA_ARGS__);          \
            fprintf(stderr, "\n");                 \
        }                                          \
    } while (0)

static void check_pack_rows(std::mt19937_64& rng) {
    for (int round = 0; round < 60; ++round) {
        const int64_t rows = 1 + static_cast<int64_t>(rng() % 700);
        const int64_t row_bytes = 1 + static_cast<int64_t>(rng() % 9000);
        const int64_t src_ld = row_bytes + static_cast<int64_t>(rng() % 3 == 0 ? 0 : rng() % 200);
        const int64_t dst_ld = row_bytes + static_cast<int64_t>(rng() % 3 == 0 ? 0 : rng() % 200);
        std::vector<uint8_t> src(static_cast<size_t>(rows * src_ld)), dst(static_cast<size_t>(rows * dst_ld), 0xAA),
            want(static_cast<size_t>(rows * dst_ld), 0xAA);
        for (auto& b : src) b = static_cast<uint8_t>(rng());
        for (int64_t r = 0; r < rows; ++r) memcpy(&want[static_cast<size_t>(r * dst_ld)], &src[static_cast<size_t>(r * src_ld)], static_cast<size_t>(row_bytes));
        const int threads = 1 + static_cast<int>(rng() % 16);
        const int rc = sh_pack_rows(dst.data(), dst_ld, src.data(), src_ld, rows, row_bytes, threads);
        EXPECT(rc == SH_OK, "sh_pack_rows rc %d", rc);
        EXPECT(dst == want, "sh_pack_rows wrote the wrong bytes (rows %lld, row_bytes %lld, threads %d)",
               static_cast<long long>(rows), static_cast<long long>(row_bytes), threads);
    }
    // a large, dense copy: the path that really splits over threads
    const int64_t rows = 4096, row_bytes = 8192;
    std::vector<uint8_t> src(static_cast<size_t>(rows * row_bytes)), dst(src.size());
    for (size_t i = 0; i < src.size(); i += 61) src[i] = static_cast<uint8_t>(i);
    EXPECT(sh_pack_rows(dst.data(), row_bytes, src.data(), row_bytes, rows, row_bytes, 8) == SH_OK, "dense pack failed");
    EXPECT(dst == src, "dense pack differs");
    uint8_t one = 0;
    EXPECT(sh_pack_rows(&one, 4, &one, 8, 2, 6, 1) == SH_ERR_INVALID_ARG, "stride shorter than a row was accepted");
    EXPECT(sh_pack_rows(nullptr, 8, &one, 8, 1, 1, 1) == SH_ERR_INVALID_ARG, "null destination was accepted");
}

static void check_sync_bytes(std::mt19937_64& rng) {
    std::vector<uint8_t> a(5000), b(5000);
    for (auto& v : a) v = static_cast<uint8_t>(rng());
    b = a;
    int32_t changed = -1;
    EXPECT(sh_sync_bytes(b.data(), a.data(), a.size(), &changed) == SH_OK && changed == 0, "equal buffers reported as different");
    a[4999] ^= 1;
    EXPECT(sh_sync_bytes(b.data(), a.data(), a.size(), &changed) == SH_OK && changed == 1 && a == b, "difference not copied");
    EXPECT(sh_sync_bytes(b.data(), a.data(), 0, &changed) == SH_OK && changed == 0, "zero bytes");
    EXPECT(sh_sync_bytes(nullptr, a.data(), 4, &changed) == SH_ERR_INVALID_ARG, "null destination was accepted");
}

static int64_t pick(std::mt19937_64& rng, int64_t bound) {
    // values that matter to a validator: around 0, around the bound, powers of two, extremes
    static const int64_t extremes[] = {0, 1, -1, 2, 15, 16, 17, 255, 256, INT64_MAX, INT64_MIN, INT64_MAX / 2, (int64_t(1) << 40),
                                       (int64_t(1) << 31), (int64_t(1) << 32) + 1, -(int64_t(1) << 40)};
    switch (rng() % 6) {
        case 0: return extremes[rng() % (sizeof(extremes) / sizeof(extremes[0]))];
        case 1: return bound + static_cast<int64_t>(rng() % 65) - 32;
        case 2: return static_cast<int64_t>(rng() % static_cast<uint64_t>(bound > 0 ? bound : 1));
        case 3: return static_cast<int64_t>(rng() % 64) * 16;
        case 4: return int64_t(1) << (rng() % 62);
        default: return static_cast<int64_t>(rng() % 4096);
    }
}

static void check_validator(std::mt19937_64& rng) {
    const size_t packed_bytes = 1 << 20, out_bytes = 2 << 20;
    std::vector<uint8_t> packed(packed_bytes), out(out_bytes);      // host memory standing in: nothing may be dereferenced
    int accepted = 0, rejected = 0, cuda = 0;
    for (int round = 0; round < 20000; ++round) {
        const int n = 1 + static_cast<int>(rng() % (round % 50 == 0 ? 300 : 6));
        std::vector<ShParamDesc> descs(static_cast<size_t>(n));
        const bool sane = rng() % 3 == 0;               // a third of the sets are well-formed, to get past the validator
        int64_t dst = 0;
        for (auto& d : descs) {
            memset(&d, 0, sizeof(d));
            if (sane) {
                d.kind = static_cast<int32_t>(rng() % 4);
                d.rows = 1 + static_cast<int64_t>(rng() % 40);
                d.cols = 16 * (1 + static_cast<int64_t>(rng() % 8));
                d.ld = d.cols + 16 * static_cast<int64_t>(rng() % 2);
                d.src_off = 256 * static_cast<int64_t>(rng() % 1000);
                d.scale_off = 512 * 1024 + 16 * static_cast<int64_t>(rng() % 1000);
                d.zp_off = rng() % 2 ? -1 : 768 * 1024 + 16 * static_cast<int64_t>(rng() % 1000);
                d.dst_off = dst;
                dst += 16 * ((d.rows * d.cols * 4 + 15) / 16);
                if (d.kind != SH_KIND_DEQUANT_I8) d.rows = 1;
            } else {
                d.kind = static_cast<int32_t>(pick(rng, 4));
                d.flags = static_cast<uint32_t>(rng() % 8);
                d.src_off = pick(rng, static_cast<int64_t>(packed_bytes));
                d.scale_off = pick(rng, static_cast<int64_t>(packed_bytes));
                d.zp_off = pick(rng, static_cast<int64_t>(packed_bytes));
                d.dst_off = pick(rng, static_cast<int64_t>(out_bytes));
                d.rows = pick(rng, 4096);
                d.cols = pick(rng, 4096);
                d.ld = pick(rng, 4096);
            }
        }
        const int32_t dtype = static_cast<int32_t>(rng() % 4);      // 3 is not a dtype
        uint64_t block = 0;
        int rc = sh_block_register(descs.data(), n, packed_bytes, out_bytes, dtype, &block);
        EXPECT(rc == SH_OK || rc == SH_ERR_INVALID_ARG || rc == SH_ERR_CUDA, "sh_block_register returned %d", rc);
        if (rc == SH_OK) sh_block_unregister(block);
        const int rc2 = sh_dequant_block_async(descs.data(), n, packed.data(), packed_bytes, out.data(), out_bytes, dtype, 0, nullptr);
        EXPECT(rc2 == SH_OK || rc2 == SH_ERR_INVALID_ARG || rc2 == SH_ERR_CUDA, "sh_dequant_block_async returned %d", rc2);
        EXPECT((rc == SH_ERR_INVALID_ARG) == (rc2 == SH_ERR_INVALID_ARG) || (descs[0].flags & SH_DESC_ABSOLUTE) || !sane,
               "the two entry points disagree on a well-formed set (%d vs %d)", rc, rc2);
        if (rc == SH_ERR_INVALID_ARG) {
            ++rejected;
            char why[256];
            EXPECT(sh_last_error(why, sizeof(why)) > 0, "a rejection without a message");
        } else if (rc == SH_ERR_CUDA) {
            ++cuda;
        } else {
            ++accepted;
        }
        if (rc != SH_ERR_INVALID_ARG) {
            // whatever got past the validator stays inside the image and the slab (offset descriptors only)
            for (const auto& d : descs) {
                if (d.flags & SH_DESC_ABSOLUTE) continue;
                const int64_t osz = dtype == SH_DT_F32 ? 4 : 2;
                if (d.kind == SH_KIND_DEQUANT_I8) {
                    EXPECT(d.src_off >= 0 && d.src_off + (d.rows - 1) * d.ld + d.cols <= static_cast<int64_t>(packed_bytes), "rows outside the image were accepted");
                    EXPECT(d.dst_off >= 0 && d.dst_off + d.rows * d.cols * osz <= static_cast<int64_t>(out_bytes), "output outside the slab was accepted");
                } else if (d.kind == SH_KIND_CAST_F32) {
                    EXPECT(d.src_off >= 0 && d.src_off + d.cols * 4 <= static_cast<int64_t>(packed_bytes), "vector outside the image was accepted");
                    EXPECT(d.dst_off >= 0 && d.dst_off + d.cols * osz <= static_cast<int64_t>(out_bytes), "output outside the slab was accepted");
                } else if (d.kind == SH_KIND_COPY || d.kind == SH_KIND_ZERO) {
                    EXPECT(d.dst_off >= 0 && d.dst_off + d.cols <= static_cast<int64_t>(out_bytes), "output outside the slab was accepted");
                }
            }
        }
    }
    printf("validator fuzz: %d sets rejected, %d past the validator (%d stopped by the CUDA runtime)\n", rejected, accepted + cuda, cuda);
    EXPECT(rejected > 1000 && accepted + cuda > 1000, "the fuzz did not exercise both outcomes");
}

int main() {
    std::mt19937_64 rng(20240611);
    check_pack_rows(rng);
    check_sync_bytes(rng);
    check_validator(rng);
    if (failures) {
        fprintf(stderr, "%d check(s) failed\n", failures);
        return 1;
    }
    printf("host checks passed\n");
    return 0;
}
