// test_mf - the reference's standalone evaluator (test_mf/test.cu:15-73) on top of libmascot:
// reads a saved model and a test file, filters the ratings the training run reported as unseen
// (unless -v 1: reconst model + reconst test set), prints "RMSE : <x>".
#include <iostream>
#include <string>
#include <sys/stat.h>
#include <vector>

#include "io_formats.h"

static bool exists(const std::string& name) {
    struct stat buffer;
    return stat(name.c_str(), &buffer) == 0;
}

int main(int argc, const char* argv[]) {
    std::string infile, testfile = "None";
    int version = 1, device = 0;
    const char* usage = " [-t <threads> -p <predictions/user> -o <output-tsv>] <input-tsv>";
    if (argc < 2) { std::cout << argv[0] << usage << std::endl; return 0; }
    if (argc == 2) infile = argv[1];
    else {
        for (int i = 0; i < argc; i++) {
            const std::string a = argv[i];
            const bool has = i < argc - 1;
            if (a == "-i" && has) infile = argv[i + 1];
            if (a == "-y" && has) testfile = argv[i + 1];
            if (a == "-v" && has) version = std::stoi(argv[i + 1]);
            if (a == "-dev" && has) device = std::stoi(argv[i + 1]);
            if (a == "-h") { std::cout << argv[0] << usage << std::endl; return 0; }
        }
    }
    if (!exists(infile)) { std::cout << infile << " doesn't exist!" << std::endl; return 0; }

    std::cout << std::endl;
    std::cout << "Input file                  : " << infile << std::endl;
    std::cout << "Test file                   : " << testfile << std::endl;
    std::cout << "Version                     : " << version << std::endl;

    std::vector<mascot_rating> test;
    if (!mascot_io::read_testset_raw(testfile, test)) { std::cout << "cannot read " << testfile << std::endl; return 1; }
    mascot_io::Model model;
    if (!mascot_io::read_model(infile, model)) { std::cout << "cannot read " << infile << std::endl; return 1; }
    if (!mascot_io::filter_removed(testfile, version, test)) return 1;

    double rmse = 0;
    const int rc = mascot_rmse_host(model.P.data(), model.n_users, model.Q.data(), model.n_items, model.k,
                                    test.data(), test.size(), device, &rmse);
    if (rc != MASCOT_OK) { std::cerr << "libmascot: " << mascot_last_error(nullptr) << std::endl; return 1; }
    std::cout << "RMSE : " << rmse << std::endl;
    return 0;
}
