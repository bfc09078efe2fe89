// quantized_mf - command line of the reference (main.cu:15-175) on top of libmascot.
//
// Same flags, defaults and output shape:
//   -i train  -y test  -o out  -l epochs(50)  -k 64|128(128)  -b lambda(0.015)  -a lr(0.01)  -d decay(0.1)
//   -wg workers  -bl block(128)  -v variant(7)  -s|-r sample ratio(0.01)  -ug / -ig groups(10)
//   -e error threshold(0.001)  -it interval(1)  -rc save reconst test set(0)
// Variants: 1 MASCOT, 2 AFP, 3 MuPPET, 4 MPT, 5 FP32 SGD, 6 MASCOT "naive" (same engine path as 1),
// 7 fp16 storage, 8 whole-model switching.
// Additive flags: -seed N, -det 1 (sequential verification mode), -dev N (first device), -g N (train on N
// GPUs of this machine: one engine and one host thread per GPU, item blocks travelling over NCCL inside
// libmascot), -bpg 1|2 (item blocks per GPU, see mascot_shard_init), -ob 1 (also write the model as a binary
// file <out>.bin / <out>_reconst.bin).  Every input file may be text or binary (cli/io_formats.h).
// Difference: when -wg is absent the engine picks the worker count itself (the reference defaults to
// 2048 warps, a setting tuned for a 36-SM GPU); the banner prints the number chosen.
#include <atomic>
#include <chrono>
#include <cmath>
#include <iostream>
#include <sstream>
#include <string>
#include <sys/stat.h>
#include <thread>
#include <vector>

#include "io_formats.h"

static bool exists(const std::string& name) {
    struct stat buffer;
    return stat(name.c_str(), &buffer) == 0;
}

namespace {

struct Run {
    mascot_config cfg;
    mascot_io::Dataset data;
    std::string infile, outfile, testfile = "None";
    unsigned reconst_save = 0, gpus = 1, blocks_per_gpu = 1, binary_out = 0;
    bool wg_given = false;
};

// Barrier of the per-GPU host threads (C++17 has none in the library).
class Barrier {
public:
    explicit Barrier(unsigned n) : n_(n) {}
    void wait() {
        const unsigned gen = gen_.load();
        if (count_.fetch_add(1) + 1 == n_) { count_.store(0); gen_.fetch_add(1); }
        else while (gen_.load() == gen) std::this_thread::yield();
    }
private:
    const unsigned n_;
    std::atomic<unsigned> count_{0}, gen_{0};
};

void print_groups(mascot_handle* h) {
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

void print_group_errors(mascot_handle* h) {                      // mf_methods.cu:327-379
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

// The timing report of mf_methods.cu:401-418, label for label (micro seconds unless stated).
void print_timings(mascot_handle* h, uint32_t epochs) {
    mascot_timings t;
    mascot_get_timings(h, &t);
    const double pre = t.rating_histogram_us + t.grouping_us + t.reconstruction_us + t.copy_to_grouped_us + t.additional_init_us;
    std::cout << "\n<Preprocessing time (micro sec)>" << std::endl;
    std::cout << "Rating histogram                 : " << t.rating_histogram_us << std::endl;
    std::cout << "Grouping                         : " << t.grouping_us << std::endl;
    std::cout << "Matrix reconstruction            : " << t.reconstruction_us << std::endl;
    std::cout << "Copy to grouped params           : " << t.copy_to_grouped_us << std::endl;
    std::cout << "Additional info init             : " << t.additional_init_us << std::endl;
    std::cout << "Total preprocessing time         : " << pre << std::endl;
    std::cout << "\n<User & item parameter copy exec time (micro sec)>" << std::endl;
    std::cout << "Precision switching              : " << t.precision_switching_us / epochs << std::endl;
    std::cout << "Total precision switching time   : " << t.precision_switching_us << std::endl;
    std::cout << "\n<User & item group error comp exec time (micro sec)>" << std::endl;
    std::cout << "Error computation time           : " << t.error_computation_us / epochs << std::endl;
    std::cout << "Total error computation time     : " << t.error_computation_us << std::endl;
    std::cout << "\n<User & item parameter update exec time (micro sec)>" << std::endl;
    std::cout << "Parameters update per epoch      : " << t.update_us / epochs << std::endl;
    std::cout << "Total parameters update          : " << t.update_us << std::endl;
    std::cout << "Total MF time(ms)                : " << (pre + t.precision_switching_us + t.error_computation_us + t.update_us) / 1000 << std::endl;
}

bool save_outputs(const Run& run, mascot_handle* h) {
    const mascot_config& cfg = run.cfg;
    const uint32_t n_users = run.data.n_users, n_items = run.data.n_items;
    if (!run.outfile.empty()) {
        std::vector<float> P((size_t)n_users * cfg.k), Q((size_t)n_items * cfg.k);
        const int order = cfg.version == MASCOT_V_MASCOT ? 1 : 0;
        if (mascot_get_factors(h, P.data(), Q.data(), order) != MASCOT_OK) return false;
        if (order == 1) {
            mascot_io::save_model_reconst(run.outfile, n_users, n_items, P.data(), Q.data(), cfg.k);
            if (run.binary_out) mascot_io::save_model_binary(run.outfile + "_reconst.bin", n_users, n_items, P.data(), Q.data(), cfg.k);
        } else {
            mascot_io::save_model(run.outfile, run.data, P.data(), Q.data(), cfg.k);
            if (run.binary_out) {
                std::vector<float> Po, Qo; uint32_t rp = 0, rq = 0;
                mascot_io::rows_in_original_order(mascot_io::orig_ids(run.data.user_orig, n_users, run.data.identity_ids), P.data(), cfg.k, Po, &rp);
                mascot_io::rows_in_original_order(mascot_io::orig_ids(run.data.item_orig, n_items, run.data.identity_ids), Q.data(), cfg.k, Qo, &rq);
                mascot_io::save_model_binary(run.outfile + ".bin", rp, rq, Po.data(), Qo.data(), cfg.k);
            }
        }
    }
    if (cfg.version == MASCOT_V_MASCOT && run.reconst_save == 1 && run.gpus == 1) {
        std::vector<mascot_rating> t(run.data.n_test);
        if (mascot_get_test_ratings(h, t.data(), 1) != MASCOT_OK) return false;
        mascot_io::save_reconst_testset(run.testfile, t);
    }
    return true;
}

int train_single(Run& run, mascot_handle* h) {
    mascot_config& cfg = run.cfg;
    auto die = [&](const char* what) {
        std::cerr << "libmascot: " << what << ": " << mascot_last_error(h) << std::endl;
        mascot_destroy(h);
        return 1;
    };
    if (cfg.version == MASCOT_V_MASCOT || cfg.version == MASCOT_V_NAIVE) print_groups(h);
    if (mascot_init_factors(h) != MASCOT_OK) return die("init_factors");
    for (uint32_t e = 0; e < cfg.epoch; e++) {
        mascot_epoch_stats st;
        if (mascot_train_epoch(h, e, &st) != MASCOT_OK) return die("train_epoch");
        if (st.error_check && (cfg.version == MASCOT_V_MASCOT || cfg.version == MASCOT_V_NAIVE)) print_group_errors(h);
        double rmse = std::nan("");                                  // no test ratings: sqrt(0 / 0), as in rmse.h:188
        if (run.data.n_test && mascot_eval_rmse(h, &rmse) != MASCOT_OK) return die("eval_rmse");
        std::cout << e + 1 << " " << st.lr << " " << rmse << std::endl;          // mf_methods.cu:396
    }
    print_timings(h, cfg.epoch);
    if (!save_outputs(run, h)) return die("writing the outputs");
    mascot_destroy(h);
    return 0;
}

// -g N: one engine and one host thread per GPU; rank 0 prints.
int train_sharded(Run& run) {
    const unsigned world = run.gpus;
    unsigned char id[MASCOT_COMM_ID_BYTES];
    if (mascot_comm_unique_id(id) != MASCOT_OK) { std::cerr << "libmascot: " << mascot_last_error(nullptr) << std::endl; return 1; }
    std::vector<mascot_handle*> hs(world, nullptr);
    std::vector<int> status(world, 0);
    std::vector<std::string> message(world);
    Barrier barrier(world);
    auto rank_main = [&](unsigned rank) {
        mascot_config cfg = run.cfg;
        cfg.device = run.cfg.device + (int)rank;
        mascot_handle* h = nullptr;
        auto failed = [&](const char* what) { status[rank] = 1; message[rank] = std::string(what) + ": " + mascot_last_error(h); };
        if (mascot_create(&cfg, &h) != MASCOT_OK) { failed("create"); return; }
        hs[rank] = h;
        if (mascot_shard_init(h, id, rank, world, run.blocks_per_gpu, 0) != MASCOT_OK) { failed("shard_init"); return; }
        if (mascot_shard_set_ratings(h, run.data.train_ptr, run.data.n_train, run.data.test_ptr, run.data.n_test, run.data.n_users, run.data.n_items) != MASCOT_OK) { failed("shard_set_ratings"); return; }
        barrier.wait();
        if (rank == 0 && (cfg.version == MASCOT_V_MASCOT || cfg.version == MASCOT_V_NAIVE)) print_groups(h);
        if (mascot_init_factors(h) != MASCOT_OK) { failed("init_factors"); return; }
        for (uint32_t e = 0; e < cfg.epoch; e++) {
            mascot_epoch_stats st;
            if (mascot_shard_train_epoch(h, e, &st) != MASCOT_OK) { failed("shard_train_epoch"); return; }
            if (rank == 0 && st.error_check) print_group_errors(h);
            double rmse = std::nan("");
            if (mascot_shard_eval_rmse(h, &rmse) != MASCOT_OK) { failed("shard_eval_rmse"); return; }
            if (!run.data.n_test) rmse = std::nan("");
            if (rank == 0) std::cout << e + 1 << " " << st.lr << " " << rmse << std::endl;
        }
        if (mascot_shard_gather_factors(h) != MASCOT_OK) { failed("shard_gather_factors"); return; }
    };
    std::vector<std::thread> threads;
    for (unsigned r = 0; r < world; r++) threads.emplace_back(rank_main, r);
    for (auto& t : threads) t.join();
    int rc = 0;
    for (unsigned r = 0; r < world; r++) if (status[r]) { std::cerr << "libmascot (GPU " << r << "): " << message[r] << std::endl; rc = 1; }
    if (!rc) {
        print_timings(hs[0], run.cfg.epoch);
        if (!save_outputs(run, hs[0])) { std::cerr << "libmascot: writing the outputs: " << mascot_last_error(hs[0]) << std::endl; rc = 1; }
    }
    // a failed run may have ranks stuck in a collective: their engines are destroyed all the same (the group is aborted)
    for (mascot_handle* h : hs) mascot_destroy(h);
    return rc;
}

}  // namespace

int main(int argc, const char* argv[]) {
    Run run;
    mascot_config& cfg = run.cfg;
    mascot_config_default(&cfg);
    const char* usage = " [-t <threads> -p <predictions/user> -o <output-tsv>] <input-tsv>";

    if (argc < 2) { std::cout << argv[0] << usage << std::endl; return 0; }
    if (argc == 2) run.infile = argv[1];
    else {
        for (int i = 0; i < argc; i++) {
            const std::string a = argv[i];
            const bool has = i < argc - 1;
            if (a == "-i" && has) run.infile = argv[i + 1];
            if (a == "-o" && has) run.outfile = argv[i + 1];
            if (a == "-y" && has) run.testfile = argv[i + 1];
            if (a == "-l" && has) cfg.epoch = (uint32_t)atoi(argv[i + 1]);
            if (a == "-k" && has) cfg.k = (uint32_t)atoi(argv[i + 1]);
            if (a == "-b" && has) cfg.lambda = (float)atof(argv[i + 1]);
            if (a == "-a" && has) cfg.learning_rate = (float)atof(argv[i + 1]);
            if (a == "-wg" && has) { cfg.num_workers = (uint32_t)atoi(argv[i + 1]); run.wg_given = true; }
            if (a == "-d" && has) cfg.decay = (float)atof(argv[i + 1]);
            if (a == "-bl" && has) cfg.thread_block_size = (uint32_t)atoi(argv[i + 1]);
            if (a == "-v" && has) cfg.version = (uint32_t)atoi(argv[i + 1]);
            if ((a == "-r" || a == "-s") && has) cfg.sample_ratio = (float)atof(argv[i + 1]);
            if (a == "-ug" && has) cfg.user_group_num = (uint32_t)atoi(argv[i + 1]);
            if (a == "-ig" && has) cfg.item_group_num = (uint32_t)atoi(argv[i + 1]);
            if (a == "-e" && has) cfg.error_threshold = (float)atof(argv[i + 1]);
            if (a == "-it" && has) cfg.interval = (uint32_t)atoi(argv[i + 1]);
            if (a == "-rc" && has) run.reconst_save = (unsigned)atoi(argv[i + 1]);
            if (a == "-seed" && has) cfg.seed = strtoull(argv[i + 1], nullptr, 10);
            if (a == "-det" && has) cfg.deterministic = (uint32_t)atoi(argv[i + 1]);
            if (a == "-dev" && has) cfg.device = atoi(argv[i + 1]);
            if (a == "-g" && has) run.gpus = (unsigned)std::max(1, atoi(argv[i + 1]));
            if (a == "-bpg" && has) run.blocks_per_gpu = (unsigned)atoi(argv[i + 1]);
            if (a == "-ob" && has) run.binary_out = (unsigned)atoi(argv[i + 1]);
            if (a == "-h") { std::cout << argv[0] << usage << std::endl; return 0; }
        }
    }
    if (!exists(run.infile)) { std::cout << run.infile << " doesn't exist!" << std::endl; return 0; }
    if (!run.wg_given) cfg.num_workers = 0;
    cfg.is_yahoo = mascot_io::is_yahoo(run.infile) ? 1u : 0u;

    // The data is read - and, on one GPU, handed to the engine - before the banner is printed: the automatic
    // worker count depends on the data.  The order of the output lines is the reference's.
    if (!mascot_io::read_training(run.data, run.infile)) { std::cout << "cannot read " << run.infile << std::endl; return 1; }
    std::ostringstream test_log;                  // what read_test prints belongs below the banner
    { std::streambuf* old = std::cout.rdbuf(test_log.rdbuf());
      const bool ok = mascot_io::read_test(run.data, run.testfile);
      std::cout.rdbuf(old);
      if (!ok) { std::cout << "cannot read " << run.testfile << std::endl; return 1; } }
    uint32_t shown_workers = cfg.num_workers;
    mascot_handle* single = nullptr;
    std::string early_error;
    if (run.gpus == 1) {
        if (mascot_create(&cfg, &single) != MASCOT_OK) early_error = mascot_last_error(nullptr);
        else if (mascot_set_ratings(single, run.data.train_ptr, run.data.n_train, run.data.test_ptr, run.data.n_test, run.data.n_users,
                                    run.data.n_items) != MASCOT_OK) early_error = std::string("set_ratings: ") + mascot_last_error(single);
        else mascot_get_worker_count(single, &shown_workers);
    } else if (!run.wg_given) {
        // the sharded engines' automatic choice (see mascot_shard_init), restated for the banner
        shown_workers = cfg.deterministic ? 1u : (uint32_t)std::max<uint64_t>(std::max<uint64_t>(run.data.n_train / 3584, 512) / run.gpus, 64);
    }
    std::cout << std::endl;
    std::cout << "Input file                  : " << run.infile << std::endl;
    std::cout << "Test file                   : " << run.testfile << std::endl;
    std::cout << "Output file                 : " << run.outfile << std::endl;
    std::cout << "Latent features             : " << cfg.k << std::endl;
    std::cout << "Learning rate               : " << cfg.learning_rate << std::endl;
    std::cout << "Decay                       : " << cfg.decay << std::endl;
    std::cout << "Lambda                      : " << cfg.lambda << std::endl;
    std::cout << "Iteration                   : " << cfg.epoch << std::endl;
    std::cout << "Num of workers              : " << shown_workers << std::endl;
    std::cout << "Thread block size           : " << cfg.thread_block_size << std::endl;
    std::cout << "Sample ratio                : " << cfg.sample_ratio << std::endl;
    std::cout << "Error threshold             : " << cfg.error_threshold << std::endl;
    std::cout << "Interval                    : " << cfg.interval << std::endl;

    std::cout << test_log.str();
    std::cout << "The number of nonzeros      : " << run.data.n_train << std::endl;
    std::cout << "The number of users         : " << run.data.n_users << std::endl;
    std::cout << "The number of items         : " << run.data.n_items << std::endl;
    std::cout << "The number of test nonzeros : " << run.data.n_test << std::endl;

    if (!early_error.empty()) { std::cerr << "libmascot: " << early_error << std::endl; mascot_destroy(single); return 1; }
    return run.gpus > 1 ? train_sharded(run) : train_single(run, single);
}
