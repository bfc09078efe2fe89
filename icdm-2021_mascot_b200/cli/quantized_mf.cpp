// quantized_mf - command line of the reference (main.cu:15-175) on top of libmascot.
//
// Same flags, defaults and output shape:
//   -i train  -y test  -o out  -l epochs(50)  -k 64|128(128)  -b lambda(0.015)  -a lr(0.01)  -d decay(0.1)
//   -wg workers  -bl block(128)  -v variant(7)  -s|-r sample ratio(0.01)  -ug / -ig groups(10)
//   -e error threshold(0.001)  -it interval(1)  -rc save reconst test set(0)
// Variants: 1 MASCOT, 2 AFP, 3 MuPPET, 4 MPT, 5 FP32 SGD, 6 MASCOT "naive" (same engine path as 1),
// 7 fp16 storage, 8 whole-model switching.  Additive flags: -seed N, -det 1 (sequential verification mode), -dev N.
// Difference: when -wg is absent the engine picks the worker count itself (the reference defaults to
// 2048 warps, a setting tuned for a 36-SM GPU).
#include <chrono>
#include <iostream>
#include <string>
#include <sys/stat.h>
#include <vector>

#include "io_formats.h"

static bool exists(const std::string& name) {
    struct stat buffer;
    return stat(name.c_str(), &buffer) == 0;
}

static double now_us() {
    return std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

int main(int argc, const char* argv[]) {
    std::string infile, outfile, testfile = "None";
    mascot_config cfg;
    mascot_config_default(&cfg);
    bool wg_given = false;
    unsigned reconst_save = 0;
    const char* usage = " [-t <threads> -p <predictions/user> -o <output-tsv>] <input-tsv>";

    if (argc < 2) { std::cout << argv[0] << usage << std::endl; return 0; }
    if (argc == 2) infile = argv[1];
    else {
        for (int i = 0; i < argc; i++) {
            const std::string a = argv[i];
            const bool has = i < argc - 1;
            if (a == "-i" && has) infile = argv[i + 1];
            if (a == "-o" && has) outfile = argv[i + 1];
            if (a == "-y" && has) testfile = argv[i + 1];
            if (a == "-l" && has) cfg.epoch = (uint32_t)atoi(argv[i + 1]);
            if (a == "-k" && has) cfg.k = (uint32_t)atoi(argv[i + 1]);
            if (a == "-b" && has) cfg.lambda = (float)atof(argv[i + 1]);
            if (a == "-a" && has) cfg.learning_rate = (float)atof(argv[i + 1]);
            if (a == "-wg" && has) { cfg.num_workers = (uint32_t)atoi(argv[i + 1]); wg_given = true; }
            if (a == "-d" && has) cfg.decay = (float)atof(argv[i + 1]);
            if (a == "-bl" && has) cfg.thread_block_size = (uint32_t)atoi(argv[i + 1]);
            if (a == "-v" && has) cfg.version = (uint32_t)atoi(argv[i + 1]);
            if ((a == "-r" || a == "-s") && has) cfg.sample_ratio = (float)atof(argv[i + 1]);
            if (a == "-ug" && has) cfg.user_group_num = (uint32_t)atoi(argv[i + 1]);
            if (a == "-ig" && has) cfg.item_group_num = (uint32_t)atoi(argv[i + 1]);
            if (a == "-e" && has) cfg.error_threshold = (float)atof(argv[i + 1]);
            if (a == "-it" && has) cfg.interval = (uint32_t)atoi(argv[i + 1]);
            if (a == "-rc" && has) reconst_save = (unsigned)atoi(argv[i + 1]);
            if (a == "-seed" && has) cfg.seed = strtoull(argv[i + 1], nullptr, 10);
            if (a == "-det" && has) cfg.deterministic = (uint32_t)atoi(argv[i + 1]);
            if (a == "-dev" && has) cfg.device = atoi(argv[i + 1]);
            if (a == "-h") { std::cout << argv[0] << usage << std::endl; return 0; }
        }
    }
    if (!exists(infile)) { std::cout << infile << " doesn't exist!" << std::endl; return 0; }
    const uint32_t shown_workers = cfg.num_workers;
    if (!wg_given) cfg.num_workers = 0;

    std::cout << std::endl;
    std::cout << "Input file                  : " << infile << std::endl;
    std::cout << "Test file                   : " << testfile << std::endl;
    std::cout << "Output file                 : " << outfile << std::endl;
    std::cout << "Latent features             : " << cfg.k << std::endl;
    std::cout << "Learning rate               : " << cfg.learning_rate << std::endl;
    std::cout << "Decay                       : " << cfg.decay << std::endl;
    std::cout << "Lambda                      : " << cfg.lambda << std::endl;
    std::cout << "Iteration                   : " << cfg.epoch << std::endl;
    if (wg_given) std::cout << "Num of workers              : " << shown_workers << std::endl;
    else std::cout << "Num of workers              : auto" << std::endl;
    std::cout << "Thread block size           : " << cfg.thread_block_size << std::endl;
    std::cout << "Sample ratio                : " << cfg.sample_ratio << std::endl;
    std::cout << "Error threshold             : " << cfg.error_threshold << std::endl;
    std::cout << "Interval                    : " << cfg.interval << std::endl;

    mascot_io::Dataset data;
    if (!mascot_io::read_training(data, infile)) { std::cout << "cannot read " << infile << std::endl; return 1; }
    if (!mascot_io::read_test(data, testfile)) { std::cout << "cannot read " << testfile << std::endl; return 1; }
    const uint32_t n_users = (uint32_t)data.user_orig.size(), n_items = (uint32_t)data.item_orig.size();
    std::cout << "The number of nonzeros      : " << data.train.size() << std::endl;
    std::cout << "The number of users         : " << n_users << std::endl;
    std::cout << "The number of items         : " << n_items << std::endl;
    std::cout << "The number of test nonzeros : " << data.test.size() << std::endl;
    cfg.is_yahoo = mascot_io::is_yahoo(infile) ? 1u : 0u;

    mascot_handle* h = nullptr;
    int rc = mascot_create(&cfg, &h);
    if (rc != MASCOT_OK) { std::cerr << "libmascot: " << mascot_last_error(nullptr) << std::endl; return 1; }
    auto die = [&](const char* what) {
        std::cerr << "libmascot: " << what << ": " << mascot_last_error(h) << std::endl;
        mascot_destroy(h);
        return 1;
    };

    const double t_pre = now_us();
    if (mascot_set_ratings(h, data.train.data(), data.train.size(), data.test.data(), data.test.size(), n_users, n_items) != MASCOT_OK)
        return die("set_ratings");
    const double preprocess_us = now_us() - t_pre;
    if (cfg.version == MASCOT_V_MASCOT || cfg.version == MASCOT_V_NAIVE) {
        for (int side = 0; side < 2; side++) {
            uint32_t ng = 0;
            mascot_get_group_info(h, side, &ng, nullptr, nullptr, nullptr);
            if (side == 0) std::cout << "The number of user groups   : " << ng << std::endl;
            else std::cout << "The number of item groups   : " << ng << std::endl;
        }
        for (int side = 0; side < 2; side++) {                       // preprocess_utils.h:192-206
            uint32_t ng = 0;
            mascot_get_group_info(h, side, &ng, nullptr, nullptr, nullptr);
            std::vector<uint32_t> end(ng);
            mascot_get_group_info(h, side, &ng, end.data(), nullptr, nullptr);
            for (uint32_t e : end) std::cout << e << " ";
            if (side == 0) std::cout << "\n\n";
        }
    }
    if (mascot_init_factors(h) != MASCOT_OK) return die("init_factors");

    double update_ms = 0, total_ms = 0;
    for (uint32_t e = 0; e < cfg.epoch; e++) {
        mascot_epoch_stats st;
        if (mascot_train_epoch(h, e, &st) != MASCOT_OK) return die("train_epoch");
        update_ms += st.kernel_ms; total_ms += st.total_ms;
        if (st.error_check) {                                        // mf_methods.cu:327-379
            for (int side = 0; side < 2; side++) {
                uint32_t ng = 0;
                mascot_get_group_info(h, side, &ng, nullptr, nullptr, nullptr);
                std::vector<float> err(ng);
                mascot_get_group_info(h, side, &ng, nullptr, nullptr, err.data());
                std::cout << (side == 0 ? "\n<User groups>\n" : "\n<Item groups>\n");
                for (float v : err) { if (v == -1) std::cout << "-1" << " "; else std::cout << v << " "; }
            }
            std::cout << "\n";
        }
        double rmse = 0;
        if (!data.test.empty() && mascot_eval_rmse(h, &rmse) != MASCOT_OK) return die("eval_rmse");
        std::cout << e + 1 << " " << st.lr << " " << rmse << std::endl;          // mf_methods.cu:396
    }

    // timing report in the shape of mf_methods.cu:401-418 (micro seconds unless stated)
    std::cout << "\n<Preprocessing time (micro sec)>" << std::endl;
    std::cout << "Total preprocessing time         : " << preprocess_us << std::endl;
    std::cout << "\n<User & item parameter update exec time (micro sec)>" << std::endl;
    std::cout << "Parameters update per epoch      : " << update_ms * 1000.0 / cfg.epoch << std::endl;
    std::cout << "Total parameters update          : " << update_ms * 1000.0 << std::endl;
    std::cout << "Total MF time(ms)                : " << preprocess_us / 1000.0 + total_ms << std::endl;

    if (!outfile.empty()) {
        std::vector<float> P((size_t)n_users * cfg.k), Q((size_t)n_items * cfg.k);
        const int order = cfg.version == MASCOT_V_MASCOT ? 1 : 0;
        if (mascot_get_factors(h, P.data(), Q.data(), order) != MASCOT_OK) return die("get_factors");
        if (order == 1) mascot_io::save_model_reconst(outfile, n_users, n_items, P.data(), Q.data(), cfg.k);
        else mascot_io::save_model(outfile, data, P.data(), Q.data(), cfg.k);
    }
    if (cfg.version == MASCOT_V_MASCOT && reconst_save == 1) {
        std::vector<mascot_rating> t(data.test.size());
        if (mascot_get_test_ratings(h, t.data(), 1) != MASCOT_OK) return die("get_test_ratings");
        mascot_io::save_reconst_testset(testfile, t);
    }
    mascot_destroy(h);
    return 0;
}
