// convert_ratings - between the rating file formats of quantized_mf / test_mf (cli/io_formats.h).
//
//   convert_ratings <in> <out.bin> bin        any readable input -> binary file (ids compacted in first-seen order
//                                             unless the input is a binary file whose ids are compact already)
//   convert_ratings <in.bin> <out> tsv        -> "user\titem\trating" lines (io_utils.h:81-83)
//   convert_ratings <in.bin> <out> item_first -> "item\tuser\trating" lines, the order the reference expects for
//                                                paths containing "netflix" or "25M" (io_utils.h:40-47)
//   convert_ratings <in.bin> <out> yahoo      -> the block format "<user>|<count>" + <count> lines "<item>\t<rating>"
//                                                (io_utils.h:49-79); ratings are written as (r - 1) * 25, the inverse
//                                                of the rescaling both programs apply to paths containing "Yahoo"
// No counterpart in the reference.  Used to feed the same synthetic set to the reference build and to this engine.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <numeric>
#include <string>
#include <vector>

#include "io_formats.h"

namespace {

// Appends the shortest decimal form that reads back as the same float.
inline char* put_float(char* p, float v) {
    if (v == std::floor(v) && std::fabs(v) < 1e7f) return p + std::sprintf(p, "%d", (int)v);
    return p + std::sprintf(p, "%.9g", (double)v);
}

struct Writer {
    FILE* f; std::vector<char> buf; size_t used = 0;
    explicit Writer(FILE* file) : f(file), buf(1 << 22) {}
    char* room(size_t n) { if (used + n > buf.size()) flush(); return buf.data() + used; }
    void flush() { if (used) std::fwrite(buf.data(), 1, used, f); used = 0; }
};

}  // namespace

int main(int argc, const char* argv[]) {
    if (argc != 4) { std::fprintf(stderr, "usage: %s <in> <out> bin|tsv|item_first|yahoo\n", argv[0]); return 2; }
    const std::string in = argv[1], out = argv[2], mode = argv[3];
    mascot_io::Dataset d;
    if (!mascot_io::read_training(d, in)) { std::fprintf(stderr, "cannot read %s\n", in.c_str()); return 1; }
    if (mode == "bin") {
        const uint32_t flags = mascot_io::kFlagCompactIds;      // what read_training returns is always compact
        if (!mascot_io::write_binary_ratings(out, d.train_ptr, d.n_train, d.n_users, d.n_items, flags)) { std::fprintf(stderr, "cannot write %s\n", out.c_str()); return 1; }
        return 0;
    }
    FILE* f = std::fopen(out.c_str(), "wb");
    if (!f) { std::fprintf(stderr, "cannot write %s\n", out.c_str()); return 1; }
    Writer w(f);
    const mascot_rating* R = d.train_ptr;
    auto orig_u = [&](uint32_t c) { return d.identity_ids ? c : d.user_orig[c]; };
    auto orig_i = [&](uint32_t c) { return d.identity_ids ? c : d.item_orig[c]; };
    if (mode == "tsv" || mode == "item_first") {
        const bool item_first = mode == "item_first";
        for (uint64_t j = 0; j < d.n_train; j++) {
            char* p = w.room(64); char* s = p;
            p += std::sprintf(p, "%u\t%u\t", item_first ? orig_i(R[j].i) : orig_u(R[j].u), item_first ? orig_u(R[j].u) : orig_i(R[j].i));
            p = put_float(p, R[j].r);
            *p++ = '\n';
            w.used += (size_t)(p - s);
        }
    } else if (mode == "yahoo") {
        // ratings grouped by user (stable: the order inside a user is the file order)
        std::vector<uint64_t> start((size_t)d.n_users + 1, 0);
        for (uint64_t j = 0; j < d.n_train; j++) start[R[j].u + 1]++;
        for (uint32_t u = 0; u < d.n_users; u++) start[u + 1] += start[u];
        std::vector<uint32_t> order(d.n_train);
        { std::vector<uint64_t> pos(start.begin(), start.end() - 1);
          for (uint64_t j = 0; j < d.n_train; j++) order[pos[R[j].u]++] = (uint32_t)j; }
        for (uint32_t u = 0; u < d.n_users; u++) {
            const uint64_t cnt = start[u + 1] - start[u];
            if (!cnt) continue;
            char* p = w.room(48); char* s = p;
            p += std::sprintf(p, "%u|%llu\n", orig_u(u), (unsigned long long)cnt);
            w.used += (size_t)(p - s);
            for (uint64_t q = start[u]; q < start[u + 1]; q++) {
                const mascot_rating& r = R[order[q]];
                p = w.room(48); s = p;
                p += std::sprintf(p, "%u\t", orig_i(r.i));
                p = put_float(p, std::nearbyint((r.r - 1.0f) * 25.0f * 1000.0f) / 1000.0f);
                *p++ = '\n';
                w.used += (size_t)(p - s);
            }
        }
    } else { std::fprintf(stderr, "unknown mode %s\n", mode.c_str()); std::fclose(f); return 2; }
    w.flush();
    return std::fclose(f) == 0 ? 0 : 1;
}
