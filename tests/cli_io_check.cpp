// Exercises cli/io_formats.h without a GPU: parses rating files, writes and re-reads model files.
// Built and driven by tests/test_cli_formats.py.
#include <cstdio>
#include <iostream>
#include "io_formats.h"

int main(int argc, char** argv) {
    if (argc < 2) return 2;
    const std::string mode = argv[1];
    if (mode == "parse" && argc >= 4) {
        mascot_io::Dataset d;
        if (!mascot_io::read_training(d, argv[2]) || !mascot_io::read_test(d, argv[3])) return 3;
        std::printf("users %zu items %zu train %zu test %zu missing %llu\n", d.user_orig.size(), d.item_orig.size(),
                    d.train.size(), d.test.size(), (unsigned long long)d.missing);
        for (size_t j = 0; j < d.train.size(); j++)
            std::printf("T %u %u %.9g %u %u\n", d.train[j].u, d.train[j].i, d.train[j].r, d.user_orig[d.train[j].u], d.item_orig[d.train[j].i]);
        for (size_t j = 0; j < d.test.size(); j++)
            std::printf("E %u %u %.9g\n", d.test[j].u, d.test[j].i, d.test[j].r);
        return 0;
    }
    if (mode == "model" && argc >= 4) {      // write a model for the parsed training file, read it back
        mascot_io::Dataset d;
        if (!mascot_io::read_training(d, argv[2])) return 3;
        const uint32_t k = 64, nu = (uint32_t)d.user_orig.size(), ni = (uint32_t)d.item_orig.size();
        std::vector<float> P((size_t)nu * k), Q((size_t)ni * k);
        for (size_t j = 0; j < P.size(); j++) P[j] = 0.001f * (float)(j % 977) - 0.3f;
        for (size_t j = 0; j < Q.size(); j++) Q[j] = 0.002f * (float)(j % 631) + 0.125f;
        if (!mascot_io::save_model(argv[3], d, P.data(), Q.data(), k)) return 4;
        if (!mascot_io::save_model_reconst(argv[3], nu, ni, P.data(), Q.data(), k)) return 4;
        mascot_io::Model m, r;
        if (!mascot_io::read_model(std::string(argv[3]) + ".txt", m)) return 5;
        if (!mascot_io::read_model(std::string(argv[3]) + "_reconst.txt", r)) return 5;
        std::printf("orig %u %u %u reconst %u %u %u\n", m.n_users, m.n_items, m.k, r.n_users, r.n_items, r.k);
        // original-id space: row of original id o equals row of its compact id; gaps are zero rows
        double err = 0, gap = 0;
        std::vector<char> seen(m.n_users, 0);
        for (uint32_t c = 0; c < nu; c++) {
            seen[d.user_orig[c]] = 1;
            for (uint32_t j = 0; j < k; j++) err = std::max(err, (double)std::abs(m.P[(size_t)d.user_orig[c] * k + j] - P[(size_t)c * k + j]));
        }
        for (uint32_t o = 0; o < m.n_users; o++) if (!seen[o]) for (uint32_t j = 0; j < k; j++) gap = std::max(gap, (double)std::abs(m.P[(size_t)o * k + j]));
        for (uint32_t c = 0; c < ni; c++)
            for (uint32_t j = 0; j < k; j++) err = std::max(err, (double)std::abs(m.Q[(size_t)d.item_orig[c] * k + j] - Q[(size_t)c * k + j]));
        for (size_t j = 0; j < P.size(); j++) err = std::max(err, (double)std::abs(r.P[j] - P[j]));
        for (size_t j = 0; j < Q.size(); j++) err = std::max(err, (double)std::abs(r.Q[j] - Q[j]));
        std::printf("max_err %.3g gap %.3g\n", err, gap);
        return 0;
    }
    if (mode == "binmodel" && argc >= 3) {   // binary model: write, read back, compare bit for bit
        const uint32_t k = 64, nu = 7, ni = 5;
        std::vector<float> P((size_t)nu * k), Q((size_t)ni * k);
        for (size_t j = 0; j < P.size(); j++) P[j] = 1.0f / (float)(j + 3);
        for (size_t j = 0; j < Q.size(); j++) Q[j] = -2.5f / (float)(j + 7);
        if (!mascot_io::save_model_binary(argv[2], nu, ni, P.data(), Q.data(), k)) return 4;
        mascot_io::Model m;
        if (!mascot_io::read_model(argv[2], m)) return 5;
        const bool same = m.n_users == nu && m.n_items == ni && m.k == k && m.P == P && m.Q == Q;
        std::printf("binmodel %s\n", same ? "identical" : "DIFFERENT");
        return same ? 0 : 6;
    }
    return 2;
}
