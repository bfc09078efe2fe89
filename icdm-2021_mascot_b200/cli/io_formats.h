// Text formats of the reference, byte-layout compatible (io_utils.h), with a parser that does not
// go through iostreams for the big files.
//
//   training / test ratings   three tab-separated tokens per line, other lines skipped
//                             (io_utils.h:81-83); item first when the path contains "netflix" or
//                             "25M" (io_utils.h:40-47); the "Yahoo" block format "<user>|<count>"
//                             followed by <count> lines "<item>\t<rating>" with ratings rescaled
//                             r/25 + 1 when the path contains "Yahoo" (io_utils.h:49-79)
//   ids                       compacted in first-seen order (io_utils.h:93-106)
//   test set                  pairs whose user or item never occurs in training are dropped and
//                             listed in remove_user.txt / remove_item.txt next to the test file
//                             (io_utils.h:122-240)
//   model  <out>.txt          "<max_user_id+1> <max_item_id+1> <k>\n", all P rows in ORIGINAL id
//                             order with zero rows for absent ids, "\n", all Q rows likewise;
//                             every value followed by one space, default ostream float formatting
//                             (io_utils.h:242-303)
//   model  <out>_reconst.txt  "<n_users> <n_items> <k>\n", P then Q in sorted-index order
//                             (io_utils.h:305-332)
//   reconst_<testfile>        the test set in sorted-index space (io_utils.h:374-405)
//
// Binary formats beside them (no counterpart in the reference; recognised by their magic, so every
// flag that takes a file accepts either kind):
//   ratings  32-byte header {u32 magic "MSCR", u32 version 1, u64 n, u32 n_users, u32 n_items,
//            u32 flags, u32 0} followed by n records {f32 r, u32 u, u32 i} - the Node of
//            common_struct.h:8-12.  flags bit 0: ids are already compact (0..n_users-1, 0..n_items-1):
//            the file is mapped into memory and handed to the library as it is, no pass over the
//            ratings on the host.  Without the bit the ids are compacted in first-seen order like text.
//   model    24-byte header {u32 magic "MSCM", u32 version 1, u32 rows_p, u32 rows_q, u32 k, u32 0}
//            followed by rows_p*k then rows_q*k floats: the same rows in the same order as the text
//            model of the same run (original-id rows with zero rows for absent ids, or sorted-index rows).
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <map>
#include <set>
#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>

#include "mascot.h"

namespace mascot_io {

constexpr uint32_t kRatingMagic = 0x5243534du;   // "MSCR"
constexpr uint32_t kModelMagic = 0x4d43534du;    // "MSCM"
constexpr uint32_t kFlagCompactIds = 1u;

struct RatingFileHeader { uint32_t magic, version; uint64_t n; uint32_t n_users, n_items, flags, reserved; };
struct ModelFileHeader { uint32_t magic, version, rows_p, rows_q, k, reserved; };
static_assert(sizeof(RatingFileHeader) == 32 && sizeof(ModelFileHeader) == 24, "file headers are packed");

// A read-only memory mapping of a whole file.
struct Mapping {
    const unsigned char* data = nullptr;
    size_t size = 0;
    Mapping() = default;
    Mapping(const Mapping&) = delete;
    Mapping& operator=(const Mapping&) = delete;
    ~Mapping() { if (data) munmap(const_cast<unsigned char*>(data), size); }
    bool open(const std::string& path) {
        const int fd = ::open(path.c_str(), O_RDONLY);
        if (fd < 0) return false;
        struct stat st;
        if (fstat(fd, &st) != 0 || st.st_size <= 0) { ::close(fd); return false; }
        void* p = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
        ::close(fd);
        if (p == MAP_FAILED) return false;
        data = static_cast<const unsigned char*>(p); size = (size_t)st.st_size;
        return true;
    }
};

inline bool has_magic(const std::string& path, uint32_t magic) {
    FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) return false;
    uint32_t m = 0;
    const bool ok = std::fread(&m, 4, 1, f) == 1 && m == magic;
    std::fclose(f);
    return ok;
}

struct Dataset {
    std::vector<mascot_rating> train, test;                // owned copies (text input, or binary input that needs compaction)
    const mascot_rating* train_ptr = nullptr; uint64_t n_train = 0;   // what to hand to the library: the vectors above
    const mascot_rating* test_ptr = nullptr; uint64_t n_test = 0;     // or a mapped binary file with compact ids
    Mapping train_map, test_map;
    bool identity_ids = false;                             // compact binary input: compact id == original id
    uint32_t n_users = 0, n_items = 0;
    std::vector<uint32_t> user_orig, item_orig;            // compact id -> original id (empty with identity_ids)
    std::unordered_map<uint32_t, uint32_t> user_map, item_map;   // original id -> compact id
    uint64_t missing = 0;                                  // test ratings dropped
};

inline std::string dir_of(const std::string& path) {
    const size_t p = path.find_last_of('/');
    return p == std::string::npos ? std::string("") : path.substr(0, p);
}
inline std::string file_of(const std::string& path) {
    const size_t p = path.find_last_of('/');
    return p == std::string::npos ? path : path.substr(p + 1);
}
inline bool item_first(const std::string& path) {
    return path.find("netflix") != std::string::npos || path.find("25M") != std::string::npos;
}
inline bool is_yahoo(const std::string& path) { return path.find("Yahoo") != std::string::npos; }

inline bool read_whole(const std::string& path, std::string& out) {
    FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) return false;
    std::fseek(f, 0, SEEK_END);
    const long sz = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    out.resize(sz > 0 ? (size_t)sz : 0);
    const size_t got = sz > 0 ? std::fread(&out[0], 1, (size_t)sz, f) : 0;
    std::fclose(f);
    out.resize(got);
    return true;
}

// One line split at `delim`: returns the number of tokens (at most 4 are recorded).
inline int split_line(const char* b, const char* e, char delim, const char* tok_b[4], const char* tok_e[4]) {
    int n = 0;
    const char* s = b;
    for (const char* p = b;; p++) {
        if (p == e || *p == delim) {
            if (n < 4) { tok_b[n] = s; tok_e[n] = p; }
            n++;
            s = p + 1;
            if (p == e) break;
        }
    }
    return n;
}
inline long tok_int(const char* b, const char* e) { return std::strtol(std::string(b, e).c_str(), nullptr, 10); }
inline float tok_float(const char* b, const char* e) { return (float)std::atof(std::string(b, e).c_str()); }

template <typename F>
inline void for_each_line(const std::string& text, F&& fn) {
    const char* p = text.data();
    const char* end = p + text.size();
    while (p < end) {
        const char* nl = (const char*)std::memchr(p, '\n', (size_t)(end - p));
        const char* le = nl ? nl : end;
        const char* e = le;
        if (e > p && e[-1] == '\r') e--;
        fn(p, e);
        p = le + 1;
    }
}

inline uint32_t compact(std::unordered_map<uint32_t, uint32_t>& map, std::vector<uint32_t>& orig, uint32_t id) {
    auto it = map.find(id);
    if (it != map.end()) return it->second;
    const uint32_t c = (uint32_t)orig.size();
    map.emplace(id, c);
    orig.push_back(id);
    return c;
}

// read_training_dataset (io_utils.h:30-120)
inline bool read_binary_ratings(const std::string& path, Mapping& map, RatingFileHeader& hdr, const mascot_rating** recs) {
    if (!map.open(path) || map.size < sizeof(RatingFileHeader)) return false;
    std::memcpy(&hdr, map.data, sizeof hdr);
    if (hdr.magic != kRatingMagic || hdr.version != 1 || map.size < sizeof hdr + hdr.n * sizeof(mascot_rating)) return false;
    *recs = reinterpret_cast<const mascot_rating*>(map.data + sizeof hdr);
    return true;
}

inline bool write_binary_ratings(const std::string& path, const mascot_rating* recs, uint64_t n, uint32_t n_users, uint32_t n_items, uint32_t flags) {
    FILE* f = std::fopen(path.c_str(), "wb");
    if (!f) return false;
    const RatingFileHeader hdr = {kRatingMagic, 1, n, n_users, n_items, flags, 0};
    bool ok = std::fwrite(&hdr, sizeof hdr, 1, f) == 1;
    if (ok && n) ok = std::fwrite(recs, sizeof(mascot_rating), n, f) == n;
    return std::fclose(f) == 0 && ok;
}

inline void finish_training(Dataset& d) {
    if (!d.train_ptr) { d.train_ptr = d.train.data(); d.n_train = d.train.size(); }
    if (!d.identity_ids) { d.n_users = (uint32_t)d.user_orig.size(); d.n_items = (uint32_t)d.item_orig.size(); }
}

inline bool read_training(Dataset& d, const std::string& path) {
    if (has_magic(path, kRatingMagic)) {
        RatingFileHeader hdr; const mascot_rating* recs = nullptr;
        if (!read_binary_ratings(path, d.train_map, hdr, &recs)) return false;
        if (hdr.flags & kFlagCompactIds) {          // mapped and handed over as it is
            d.identity_ids = true; d.n_users = hdr.n_users; d.n_items = hdr.n_items;
            d.train_ptr = recs; d.n_train = hdr.n;
        } else {
            d.train.reserve(hdr.n);
            for (uint64_t j = 0; j < hdr.n; j++)
                d.train.push_back({recs[j].r, compact(d.user_map, d.user_orig, recs[j].u), compact(d.item_map, d.item_orig, recs[j].i)});
        }
        finish_training(d);
        return true;
    }
    std::string text;
    if (!read_whole(path, text)) return false;
    const bool yahoo = is_yahoo(path);
    const int ui = item_first(path) ? 1 : 0, ii = item_first(path) ? 0 : 1;
    const char *tb[4], *te[4];
    if (yahoo) {
        long remaining = 0; uint32_t user_c = 0;
        for_each_line(text, [&](const char* b, const char* e) {
            if (remaining == 0) {
                if (split_line(b, e, '|', tb, te) < 2) return;
                user_c = compact(d.user_map, d.user_orig, (uint32_t)tok_int(tb[0], te[0]));
                remaining = tok_int(tb[1], te[1]);
            } else {
                remaining--;
                if (split_line(b, e, '\t', tb, te) < 2) return;
                const uint32_t item_c = compact(d.item_map, d.item_orig, (uint32_t)tok_int(tb[0], te[0]));
                d.train.push_back({tok_float(tb[1], te[1]) / 25.f + 1.0f, user_c, item_c});
            }
        });
    } else {
        for_each_line(text, [&](const char* b, const char* e) {
            if (split_line(b, e, '\t', tb, te) != 3) return;
            const uint32_t user_c = compact(d.user_map, d.user_orig, (uint32_t)tok_int(tb[ui], te[ui]));
            const uint32_t item_c = compact(d.item_map, d.item_orig, (uint32_t)tok_int(tb[ii], te[ii]));
            d.train.push_back({tok_float(tb[2], te[2]), user_c, item_c});
        });
    }
    finish_training(d);
    return true;
}

// read_test_dataset (io_utils.h:122-240).  The reference keeps the test set in a map per user, so a
// repeated (user, item) pair keeps its last rating; the result is ordered by (user, item).
inline bool read_test(Dataset& d, const std::string& path) {
    d.test_ptr = nullptr; d.n_test = 0;
    if (has_magic(path, kRatingMagic)) {
        RatingFileHeader hdr; const mascot_rating* recs = nullptr;
        if (!read_binary_ratings(path, d.test_map, hdr, &recs)) return false;
        if ((hdr.flags & kFlagCompactIds) && d.identity_ids) {       // same id space as the training file by construction
            d.test_ptr = recs; d.n_test = hdr.n;
            return true;
        }
        for (uint64_t j = 0; j < hdr.n; j++) {
            uint32_t u = recs[j].u, i = recs[j].i;
            if (d.identity_ids) { if (u >= d.n_users || i >= d.n_items) { d.missing++; continue; } }
            else {
                auto iu = d.user_map.find(u); auto it = d.item_map.find(i);
                if (iu == d.user_map.end() || it == d.item_map.end()) { d.missing++; continue; }
                u = iu->second; i = it->second;
            }
            d.test.push_back({recs[j].r, u, i});
        }
        std::cout << "Missing the number of ratings : " << d.missing << std::endl;
        d.test_ptr = d.test.data(); d.n_test = d.test.size();
        return true;
    }
    std::string text;
    // a missing test file (the default "None") is an empty test set, like the reference, whose ifstream
    // simply yields no lines (io_utils.h:131-132)
    if (!read_whole(path, text)) return true;
    const bool yahoo = is_yahoo(path);
    const int ui = item_first(path) ? 1 : 0, ii = item_first(path) ? 0 : 1;
    std::vector<uint32_t> remove_user, remove_item;
    std::vector<mascot_rating> raw;
    const char *tb[4], *te[4];
    if (yahoo) {
        long remaining = 0; bool known_user = false; uint32_t user_c = 0;
        for_each_line(text, [&](const char* b, const char* e) {
            if (remaining == 0) {
                if (split_line(b, e, '|', tb, te) < 2) return;
                auto it = d.user_map.find((uint32_t)tok_int(tb[0], te[0]));
                remaining = tok_int(tb[1], te[1]);
                known_user = it != d.user_map.end();
                if (known_user) user_c = it->second; else d.missing += (uint64_t)remaining;
            } else {
                remaining--;
                if (!known_user) return;
                if (split_line(b, e, '\t', tb, te) < 2) return;
                auto it = d.item_map.find((uint32_t)tok_int(tb[0], te[0]));
                if (it == d.item_map.end()) { d.missing++; return; }
                raw.push_back({tok_float(tb[1], te[1]) / 25.f + 1.0f, user_c, it->second});
            }
        });
    } else {
        for_each_line(text, [&](const char* b, const char* e) {
            if (split_line(b, e, '\t', tb, te) != 3) return;
            const uint32_t user = (uint32_t)tok_int(tb[ui], te[ui]), item = (uint32_t)tok_int(tb[ii], te[ii]);
            auto iu = d.user_map.find(user);
            auto it = d.item_map.find(item);
            if (iu != d.user_map.end() && it != d.item_map.end()) raw.push_back({tok_float(tb[2], te[2]), iu->second, it->second});
            else if (iu == d.user_map.end()) { d.missing++; remove_user.push_back(user); }
            else { d.missing++; remove_item.push_back(item); }
        });
    }
    std::stable_sort(raw.begin(), raw.end(), [](const mascot_rating& a, const mascot_rating& b) {
        return a.u != b.u ? a.u < b.u : a.i < b.i;
    });
    d.test.clear();
    for (size_t j = 0; j < raw.size(); j++) {
        if (j + 1 < raw.size() && raw[j + 1].u == raw[j].u && raw[j + 1].i == raw[j].i) continue;   // last one wins
        d.test.push_back(raw[j]);
    }
    std::cout << "Missing the number of ratings : " << d.missing << std::endl;
    const std::string dir = dir_of(path);
    for (int which = 0; which < 2; which++) {
        const std::string out = dir + (which == 0 ? "/remove_user.txt" : "/remove_item.txt");
        std::ofstream f(out.c_str(), std::ofstream::out);
        if (f.fail()) { std::cout << "fail to write file named " << out << std::endl; break; }
        for (uint32_t v : (which == 0 ? remove_user : remove_item)) f << v << std::endl;
    }
    d.test_ptr = d.test.data(); d.n_test = d.test.size();
    return true;
}

inline void write_rows_original_order(std::ofstream& f, const std::vector<uint32_t>& orig, const float* M, uint32_t k) {
    std::vector<std::pair<uint32_t, uint32_t>> order(orig.size());
    for (uint32_t c = 0; c < orig.size(); c++) order[c] = {orig[c], c};
    std::sort(order.begin(), order.end());
    uint32_t prev = 0;
    std::ostringstream buf;
    for (auto& oc : order) {
        for (uint32_t gap = prev; gap < oc.first; gap++)
            for (uint32_t j = 0; j < k; j++) buf << 0 << " ";
        for (uint32_t j = 0; j < k; j++) buf << M[(size_t)oc.second * k + j] << " ";
        prev = oc.first + 1;
        if (buf.tellp() > (1 << 20)) { f << buf.str(); buf.str(""); }
    }
    f << buf.str();
}

inline std::vector<uint32_t> orig_ids(const std::vector<uint32_t>& orig, uint32_t n, bool identity) {
    if (!identity) return orig;
    std::vector<uint32_t> v(n);
    for (uint32_t e = 0; e < n; e++) v[e] = e;
    return v;
}

// save_trained_model (io_utils.h:242-303)
inline bool save_model(const std::string& outfile, const Dataset& d, const float* P, const float* Q, uint32_t k) {
    std::cout << "Save trained model..." << std::endl;
    const std::string path = outfile + ".txt";
    std::ofstream f(path.c_str());
    if (f.fail()) { std::cout << "fail to write file named " << path << std::endl; std::cerr << "Error: " << std::strerror(errno); return false; }
    const std::vector<uint32_t> uo = orig_ids(d.user_orig, d.n_users, d.identity_ids), io = orig_ids(d.item_orig, d.n_items, d.identity_ids);
    const uint32_t max_user = *std::max_element(uo.begin(), uo.end());
    const uint32_t max_item = *std::max_element(io.begin(), io.end());
    f << max_user + 1 << " " << max_item + 1 << " " << k << std::endl;
    write_rows_original_order(f, uo, P, k);
    f << std::endl;
    write_rows_original_order(f, io, Q, k);
    return true;
}

// The binary model beside the text one: same rows, same order (see the head of this file).
inline bool save_model_binary(const std::string& path, uint32_t rows_p, uint32_t rows_q, const float* P, const float* Q, uint32_t k) {
    FILE* f = std::fopen(path.c_str(), "wb");
    if (!f) { std::cout << "fail to write file named " << path << std::endl; return false; }
    const ModelFileHeader hdr = {kModelMagic, 1, rows_p, rows_q, k, 0};
    bool ok = std::fwrite(&hdr, sizeof hdr, 1, f) == 1;
    ok = ok && std::fwrite(P, sizeof(float), (size_t)rows_p * k, f) == (size_t)rows_p * k;
    ok = ok && std::fwrite(Q, sizeof(float), (size_t)rows_q * k, f) == (size_t)rows_q * k;
    return std::fclose(f) == 0 && ok;
}

// Original-id rows with zero rows for absent ids, as save_trained_model lays them out.
inline void rows_in_original_order(const std::vector<uint32_t>& orig, const float* M, uint32_t k, std::vector<float>& out, uint32_t* rows) {
    const uint32_t max_id = *std::max_element(orig.begin(), orig.end());
    out.assign((size_t)(max_id + 1) * k, 0.f);
    for (uint32_t c = 0; c < orig.size(); c++) std::memcpy(&out[(size_t)orig[c] * k], M + (size_t)c * k, sizeof(float) * k);
    *rows = max_id + 1;
}

// save_trained_model_reconst (io_utils.h:305-332)
inline bool save_model_reconst(const std::string& outfile, uint32_t n_users, uint32_t n_items, const float* P, const float* Q, uint32_t k) {
    std::cout << "Save trained reconst model..." << std::endl;
    const std::string path = outfile + "_reconst.txt";
    std::ofstream f(path.c_str());
    if (f.fail()) { std::cout << "fail to write file named " << path << std::endl; std::cerr << "Error: " << std::strerror(errno); return false; }
    f << n_users << " " << n_items << " " << k << std::endl;
    auto dump = [&](const float* M, size_t count) {
        std::ostringstream buf;
        for (size_t j = 0; j < count; j++) {
            buf << M[j] << " ";
            if (buf.tellp() > (1 << 20)) { f << buf.str(); buf.str(""); }
        }
        f << buf.str();
    };
    dump(P, (size_t)n_users * k);
    f << std::endl;
    dump(Q, (size_t)n_items * k);
    return true;
}

// save_reconst_testset (io_utils.h:374-405)
inline bool save_reconst_testset(const std::string& testfile, const std::vector<mascot_rating>& test_sorted_space) {
    std::cout << "Save reconst mat.." << std::endl;
    const std::string path = dir_of(testfile) + "/reconst_" + file_of(testfile);
    std::ofstream f(path.c_str(), std::ofstream::out);
    if (f.fail()) { std::cout << "fail to write file named " << path << std::endl; return false; }
    const bool user_first = !item_first(path);
    for (const mascot_rating& t : test_sorted_space) {
        if (user_first) f << t.u << "\t" << t.i << "\t" << t.r << std::endl;
        else f << t.i << "\t" << t.u << "\t" << t.r << std::endl;
    }
    return true;
}

struct Model {
    uint32_t n_users = 0, n_items = 0, k = 0;
    std::vector<float> P, Q;
};

// read_trained_model (io_utils.h:334-372): header tokens, then whitespace-separated floats
inline bool read_model(const std::string& path, Model& m) {
    if (has_magic(path, kModelMagic)) {
        Mapping map;
        ModelFileHeader hdr;
        if (!map.open(path) || map.size < sizeof hdr) return false;
        std::memcpy(&hdr, map.data, sizeof hdr);
        const size_t np = (size_t)hdr.rows_p * hdr.k, nq = (size_t)hdr.rows_q * hdr.k;
        if (hdr.version != 1 || map.size < sizeof hdr + (np + nq) * sizeof(float)) return false;
        m.n_users = hdr.rows_p; m.n_items = hdr.rows_q; m.k = hdr.k;
        const float* v = reinterpret_cast<const float*>(map.data + sizeof hdr);
        m.P.assign(v, v + np); m.Q.assign(v + np, v + np + nq);
        return true;
    }
    std::string text;
    if (!read_whole(path, text)) return false;
    char* p = &text[0];
    char* end = nullptr;
    m.n_users = (uint32_t)std::strtoul(p, &end, 10); p = end;
    m.n_items = (uint32_t)std::strtoul(p, &end, 10); p = end;
    m.k = (uint32_t)std::strtoul(p, &end, 10); p = end;
    m.P.resize((size_t)m.n_users * m.k);
    m.Q.resize((size_t)m.n_items * m.k);
    for (float& v : m.P) { v = std::strtof(p, &end); if (end == p) return false; p = end; }
    for (float& v : m.Q) { v = std::strtof(p, &end); if (end == p) return false; p = end; }
    return true;
}

// read_testset_pretrained_model (io_utils.h:407-456): ids are used as they stand in the file
inline bool read_testset_raw(const std::string& path, std::vector<mascot_rating>& out) {
    if (has_magic(path, kRatingMagic)) {
        Mapping map; RatingFileHeader hdr; const mascot_rating* recs = nullptr;
        if (!read_binary_ratings(path, map, hdr, &recs)) return false;
        out.assign(recs, recs + hdr.n);
        return true;
    }
    std::string text;
    if (!read_whole(path, text)) return false;
    const int ui = item_first(path) ? 1 : 0, ii = item_first(path) ? 0 : 1;
    const char *tb[4], *te[4];
    if (is_yahoo(path) && path.find("reconst") == std::string::npos) {
        long remaining = 0; uint32_t user = 0;
        for_each_line(text, [&](const char* b, const char* e) {
            if (remaining == 0) {
                if (split_line(b, e, '|', tb, te) < 2) return;
                user = (uint32_t)tok_int(tb[0], te[0]);
                remaining = tok_int(tb[1], te[1]);
            } else {
                remaining--;
                if (split_line(b, e, '\t', tb, te) < 2) return;
                out.push_back({tok_float(tb[1], te[1]) / 25.f + 1.0f, user, (uint32_t)tok_int(tb[0], te[0])});
            }
        });
    } else {
        for_each_line(text, [&](const char* b, const char* e) {
            if (split_line(b, e, '\t', tb, te) != 3) return;
            out.push_back({tok_float(tb[2], te[2]), (uint32_t)tok_int(tb[ui], te[ui]), (uint32_t)tok_int(tb[ii], te[ii])});
        });
    }
    return true;
}

// remove_elements (io_utils.h:458-515): for models in original-id space, drop the test ratings whose
// user or item was listed as unseen when the training run read this test file
inline bool filter_removed(const std::string& testfile, int version, std::vector<mascot_rating>& test) {
    if (version == 1) return true;
    std::set<uint32_t> ru, ri;
    const std::string dir = dir_of(testfile);
    for (int which = 0; which < 2; which++) {
        const std::string path = dir + (which == 0 ? "/remove_user.txt" : "/remove_item.txt");
        std::ifstream f(path.c_str());
        if (f.fail()) { std::cout << "fail to write file named " << path << std::endl; return false; }
        std::string line;
        while (std::getline(f, line)) {
            if (line.empty()) continue;
            (which == 0 ? ru : ri).insert((uint32_t)std::strtoul(line.c_str(), nullptr, 10));
        }
    }
    std::vector<mascot_rating> kept;
    for (const mascot_rating& t : test)
        if (!ru.count(t.u) && !ri.count(t.i)) kept.push_back(t);
    test.swap(kept);
    return true;
}

}  // namespace mascot_io
