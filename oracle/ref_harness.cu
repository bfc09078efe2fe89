// Reference-kernel harness: TEST INFRASTRUCTURE ONLY, never linked into the product.
//
// Compiled against the reference's own kernel headers where they lie (passed with -I at build
// time; nothing of the reference is copied into this repository), it launches each reference
// training kernel with ONE warp on tiny seeded problems and dumps the resulting factors and
// statistics.  The cuRAND state is seeded with a fixed value and a probe kernel records the
// chunk start positions the training kernel will draw, so a CPU replay can follow exactly the
// same sequence of updates.  The outputs become golden vectors for the CPU oracle.
// Cases of kind 8 run the reference's m-quantization set-up instead (degree histogram and sort,
// grouping, index maps, remapped ratings, scatter of the factors into the per-group binary16
// arenas) through the reference's own host functions and dump every table they produce.
//
// usage: ref_harness <harness_in.bin> <harness_out.bin>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cstdint>
#include <cmath>
#include <map>
#include <string>
#include <vector>
#include <iostream>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <curand_kernel.h>

#include <thrust/device_ptr.h>
#include <thrust/sort.h>

#include "common.h"
#include "common_struct.h"
#include "preprocess_utils.h"
#include "model_init.h"
#include "reduce_kernel.h"
#include "sgd_kernel.h"
#include "sgd_kernel_k64.h"
#include "mascot_sgd_kernel.h"
#include "mascot_sgd_kernel_k64.h"
#include "mpt_sgd_kernel.h"
#include "mpt_sgd_kernel_k64.h"
#include "muppet_sgd_kernel.h"
#include "muppet_sgd_kernel_k64.h"
#include "afp_sgd_kernel.h"
#include "afp_sgd_kernel_k64.h"
#include "rmse.h"

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { \
    fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); exit(2); } } while (0)

struct Entry { uint32_t dtype; std::vector<char> data; uint64_t n; };
typedef std::map<std::string, Entry> Bundle;
static const size_t kDtSize[] = {4, 4, 4, 2, 1, 8};

static Bundle read_bundle(const char* path) {
    Bundle b;
    FILE* f = fopen(path, "rb");
    if (!f) { fprintf(stderr, "cannot open %s\n", path); exit(2); }
    char magic[4]; uint32_t count;
    if (fread(magic, 1, 4, f) != 4 || memcmp(magic, "MSCB", 4) || fread(&count, 4, 1, f) != 1) exit(2);
    for (uint32_t e = 0; e < count; e++) {
        char name[48]; uint32_t hdr[2]; uint64_t n;
        if (fread(name, 1, 48, f) != 48 || fread(hdr, 4, 2, f) != 2 || fread(&n, 8, 1, f) != 1) exit(2);
        Entry en; en.dtype = hdr[0]; en.n = n;
        size_t nb = n * kDtSize[hdr[0]];
        en.data.resize(nb);
        if (nb && fread(en.data.data(), 1, nb, f) != nb) exit(2);
        fseek(f, (long)((8 - nb % 8) % 8), SEEK_CUR);
        b[std::string(name)] = en;
    }
    fclose(f);
    return b;
}

static void put(Bundle& b, const std::string& name, uint32_t dtype, const void* p, uint64_t n) {
    Entry en; en.dtype = dtype; en.n = n;
    en.data.assign((const char*)p, (const char*)p + n * kDtSize[dtype]);
    b[name] = en;
}

static void write_bundle(const char* path, const Bundle& b) {
    FILE* f = fopen(path, "wb");
    if (!f) { fprintf(stderr, "cannot write %s\n", path); exit(2); }
    uint32_t count = (uint32_t)b.size();
    fwrite("MSCB", 1, 4, f); fwrite(&count, 4, 1, f);
    for (auto& kv : b) {
        char name[48]; memset(name, 0, 48); strncpy(name, kv.first.c_str(), 47);
        uint32_t hdr[2] = {kv.second.dtype, 0};
        fwrite(name, 1, 48, f); fwrite(hdr, 4, 2, f); fwrite(&kv.second.n, 8, 1, f);
        size_t nb = kv.second.data.size();
        if (nb) fwrite(kv.second.data.data(), 1, nb, f);
        char pad[8] = {0}; fwrite(pad, 1, (8 - nb % 8) % 8, f);
    }
    fclose(f);
}

template <typename T> static const T* get(const Bundle& b, const std::string& name, uint64_t* n = nullptr) {
    auto it = b.find(name);
    if (it == b.end()) { fprintf(stderr, "missing entry %s\n", name.c_str()); exit(2); }
    if (n) *n = it->second.n;
    return (const T*)it->second.data.data();
}

__global__ void seed_state(curandState* st, int seed) { curand_init(seed, 0, 0, &st[0]); }

// Draw the chunk starts exactly the way every reference training kernel does, on a COPY of the state.
__global__ void probe_starts(const curandState* st, unsigned int nnz, int count, unsigned int* out) {
    curandState s = st[0];
    for (int c = 0; c < count; c++) {
        unsigned int origin = (unsigned int)(curand_uniform(&s) * nnz);
        out[c] = origin % nnz;
    }
}

template <typename T> static T* to_dev(const T* h, size_t n) {
    T* d; CK(cudaMalloc(&d, sizeof(T) * (n ? n : 1)));
    if (n) CK(cudaMemcpy(d, h, sizeof(T) * n, cudaMemcpyHostToDevice));
    return d;
}


// kind 8: the reference's set-up pipeline of mascot_training_mf (mf_methods.cu:41-90) on a small
// seeded rating set: user_item_rating_histogram, split_group_based_equal_size_not_strict_ret_end_idx,
// matrix_reconstruction (preprocess_utils.h:54-255) and cpy2grouped_parameters_gpu_for_comparison_indexing
// (model_init.cu:175-222), called as they are.
static void run_setup_case(const Bundle& in, Bundle& out, const std::string& name) {
    const int* meta = get<int>(in, name + ".meta");
    const int k = meta[1], n_users = meta[2], n_items = meta[3], nnz = meta[4], n_test = meta[5];
    const int ug_req = meta[6], ig_req = meta[7];
    const Node* R = (const Node*)get<uint32_t>(in, name + ".R");
    const Node* T = (const Node*)get<uint32_t>(in, name + ".T");
    const float* P = get<float>(in, name + ".P");
    const float* Q = get<float>(in, name + ".Q");
    Mf_info mf;
    SGD sgd;
    mf.max_user = n_users; mf.max_item = n_items; mf.n = nnz; mf.test_n = n_test;
    mf.params.k = k; mf.params.user_group_num = ug_req; mf.params.item_group_num = ig_req;
    mf.d_R = to_dev(R, nnz);
    mf.d_test_COO = to_dev(T, n_test);
    user_item_rating_histogram(&mf);
    put(out, name + ".user2cnt", 1, mf.user2cnt, n_users); put(out, name + ".item2cnt", 1, mf.item2cnt, n_items);
    put(out, name + ".user2idx", 1, mf.user2idx, n_users); put(out, name + ".item2idx", 1, mf.item2idx, n_items);
    split_group_based_equal_size_not_strict_ret_end_idx(&mf);
    std::cout << std::endl;
    const unsigned ug = mf.params.user_group_num, ig = mf.params.item_group_num;
    put(out, name + ".uend", 1, mf.user_group_end_idx, ug); put(out, name + ".iend", 1, mf.item_group_end_idx, ig);
    put(out, name + ".user_group_idx", 1, mf.user_group_idx, n_users); put(out, name + ".item_group_idx", 1, mf.item_group_idx, n_items);
    matrix_reconstruction(&mf);
    put(out, name + ".user2sorted", 1, mf.user2sorted_idx, n_users); put(out, name + ".item2sorted", 1, mf.item2sorted_idx, n_items);
    put(out, name + ".user_group_size", 1, mf.user_group_size, ug); put(out, name + ".item_group_size", 1, mf.item_group_size, ig);
    std::vector<Node> Rm(nnz), Tm(n_test);
    CK(cudaMemcpy(Rm.data(), mf.d_R, sizeof(Node) * nnz, cudaMemcpyDeviceToHost));
    if (n_test) CK(cudaMemcpy(Tm.data(), mf.d_test_COO, sizeof(Node) * n_test, cudaMemcpyDeviceToHost));
    put(out, name + ".R_sorted_ids", 1, Rm.data(), (uint64_t)nnz * 3); put(out, name + ".T_sorted_ids", 1, Tm.data(), (uint64_t)n_test * 3);
    // scatter into the per-group binary16 arenas (mf_methods.cu:80-90 allocates the pointer tables)
    sgd.d_p = to_dev(P, (size_t)n_users * k); sgd.d_q = to_dev(Q, (size_t)n_items * k);
    CK(cudaMallocHost(&sgd.user_group_d_ptr, sizeof(void*) * ug)); CK(cudaMallocHost(&sgd.item_group_d_ptr, sizeof(void*) * ig));
    CK(cudaMallocHost(&sgd.user_group_ptr, sizeof(void*) * ug)); CK(cudaMallocHost(&sgd.item_group_ptr, sizeof(void*) * ig));
    CK(cudaMalloc(&sgd.d_user_group_ptr, sizeof(void*) * ug)); CK(cudaMalloc(&sgd.d_item_group_ptr, sizeof(void*) * ig));
    cpy2grouped_parameters_gpu_for_comparison_indexing(&mf, &sgd);
    auto fetch = [&](void** dptr, const unsigned int* size, unsigned groups, size_t rows, const std::string& key) {
        std::vector<float> all(rows * k);
        size_t row0 = 0;
        for (unsigned g = 0; g < groups; g++) {
            const size_t cnt = (size_t)size[g] * k;
            std::vector<__half> h(cnt);
            if (cnt) CK(cudaMemcpy(h.data(), dptr[g], sizeof(__half) * cnt, cudaMemcpyDeviceToHost));
            for (size_t j = 0; j < cnt; j++) all[row0 * k + j] = __half2float(h[j]);
            row0 += size[g];
        }
        put(out, name + key, 0, all.data(), rows * k);
    };
    fetch(sgd.user_group_d_ptr, mf.user_group_size, ug, n_users, ".P_arena");
    fetch(sgd.item_group_d_ptr, mf.item_group_size, ig, n_items, ".Q_arena");
    printf("case %-22s set-up: users %d items %d nnz %d groups %u/%u\n", name.c_str(), n_users, n_items, nnz, ug, ig);
}

int main(int argc, char** argv) {
    if (argc < 3) { fprintf(stderr, "usage: %s in.bin out.bin\n", argv[0]); return 2; }
    Bundle in = read_bundle(argv[1]);
    Bundle out;
    uint64_t ncs; const char* cs = get<char>(in, "cases", &ncs);
    std::string all(cs, cs + ncs);
    std::vector<std::string> cases;
    size_t pos = 0;
    while (pos <= all.size()) {
        size_t nl = all.find('\n', pos);
        if (nl == std::string::npos) nl = all.size();
        if (nl > pos) cases.push_back(all.substr(pos, nl - pos));
        pos = nl + 1;
    }

    for (auto& name : cases) {
        const int* meta = get<int>(in, name + ".meta");
        if (meta[0] == 8) { run_setup_case(in, out, name); continue; }
        const float* hyper = get<float>(in, name + ".hyper");
        int kind = meta[0], k = meta[1], n_users = meta[2], n_items = meta[3], nnz = meta[4];
        int update_count = meta[5], vec = meta[6], first_sample = meta[7], seed = meta[8], extra0 = meta[9];
        float lr = hyper[0], lam = hyper[1];
        const Node* R = (const Node*)get<uint32_t>(in, name + ".R");
        const float* P = get<float>(in, name + ".P");
        const float* Q = get<float>(in, name + ".Q");
        size_t np = (size_t)n_users * k, nq = (size_t)n_items * k;
        Node* dR = to_dev(R, nnz);
        std::vector<float> Pout(np), Qout(nq);
        printf("case %-22s kind %d k %d users %d items %d nnz %d\n", name.c_str(), kind, k, n_users, n_items, nnz);

        if (kind == 6) {  // test RMSE
            float* dP = to_dev(P, np); float* dQ = to_dev(Q, nq);
            unsigned int groups = (unsigned int)ceil(nnz / (float)512);
            unsigned int iter_num = (unsigned int)ceil(nnz / (float)(512 * groups));
            float* dE; CK(cudaMalloc(&dE, sizeof(float) * groups));
            if (k == 128) get_test_rmse_coalesced_k128<<<groups, 512>>>(dR, dP, dQ, dE, iter_num, 32, nnz, k);
            else get_test_rmse_coalesced_k64<<<groups, 512>>>(dR, dP, dQ, dE, iter_num, 32, nnz, k);
            CK(cudaDeviceSynchronize());
            std::vector<float> e(groups);
            CK(cudaMemcpy(e.data(), dE, sizeof(float) * groups, cudaMemcpyDeviceToHost));
            float sum = 0; for (unsigned int g = 0; g < groups; g++) sum += e[g];
            float rmse = sqrt(sum / (double)nnz);
            put(out, name + ".group_err", 0, e.data(), groups);
            put(out, name + ".rmse", 0, &rmse, 1);
            cudaFree(dP); cudaFree(dQ); cudaFree(dE); cudaFree(dR);
            continue;
        }

        curandState* dState; CK(cudaMalloc(&dState, sizeof(curandState)));
        seed_state<<<1, 1>>>(dState, seed);
        unsigned int* dStarts; CK(cudaMalloc(&dStarts, sizeof(unsigned int) * update_count));
        probe_starts<<<1, 1>>>(dState, nnz, update_count, dStarts);
        CK(cudaDeviceSynchronize());
        std::vector<unsigned int> starts(update_count);
        CK(cudaMemcpy(starts.data(), dStarts, sizeof(unsigned int) * update_count, cudaMemcpyDeviceToHost));
        put(out, name + ".start_ids", 1, starts.data(), update_count);

        if (kind == 1) {  // MASCOT: grouped fp16/fp32 arenas
            uint64_t ug, ig;
            const unsigned int* uend = get<unsigned int>(in, name + ".uend", &ug);
            const unsigned int* iend = get<unsigned int>(in, name + ".iend", &ig);
            const unsigned char* uprec = get<unsigned char>(in, name + ".uprec");
            const unsigned char* iprec = get<unsigned char>(in, name + ".iprec");
            auto build = [&](const float* M, const unsigned int* end, const unsigned char* prec, int groups,
                             std::vector<void*>& ptrs) {
                int start = 0;
                for (int g = 0; g < groups; g++) {
                    size_t cnt = (size_t)(end[g] + 1 - start) * k;
                    void* d;
                    if (prec[g]) { d = to_dev(M + (size_t)start * k, cnt); }
                    else {
                        std::vector<__half> h(cnt);
                        for (size_t j = 0; j < cnt; j++) h[j] = __float2half_rn(M[(size_t)start * k + j]);
                        d = to_dev(h.data(), cnt);
                    }
                    ptrs.push_back(d);
                    start = end[g] + 1;
                }
            };
            std::vector<void*> up, ip;
            build(P, uend, uprec, (int)ug, up); build(Q, iend, iprec, (int)ig, ip);
            void** dUp = to_dev(up.data(), ug); void** dIp = to_dev(ip.data(), ig);
            unsigned int* dUend = to_dev(uend, ug); unsigned int* dIend = to_dev(iend, ig);
            unsigned char* dUprec = to_dev(uprec, ug); unsigned char* dIprec = to_dev(iprec, ig);
            float *dGp, *dGq, *dNp, *dNq;
            CK(cudaMalloc(&dGp, sizeof(float) * ug * k)); CK(cudaMemset(dGp, 0, sizeof(float) * ug * k));
            CK(cudaMalloc(&dGq, sizeof(float) * ig * k)); CK(cudaMemset(dGq, 0, sizeof(float) * ig * k));
            CK(cudaMalloc(&dNp, sizeof(float) * ug)); CK(cudaMalloc(&dNq, sizeof(float) * ig));
            size_t smem = 16384;  // generous: the reference sizes this a few bytes short for > 62 groups
            if (k == 128)
                mascot_sgd_k128_hogwild_kernel<<<1, 32, smem>>>(dR, nnz, dUp, dIp, dState, lr, k, update_count, vec, lam,
                    dUend, dIend, dUprec, dIprec, dGp, dGq, dNp, dNq, first_sample, (int)ug, (int)ig);
            else
                mascot_sgd_k64_hogwild_kernel<<<1, 32, smem>>>(dR, nnz, dUp, dIp, dState, lr, k, update_count, vec, lam,
                    dUend, dIend, dUprec, dIprec, dGp, dGq, dNp, dNq, first_sample, (int)ug, (int)ig);
            CK(cudaDeviceSynchronize());
            auto fetch = [&](float* M, const unsigned int* end, const unsigned char* prec, int groups,
                             std::vector<void*>& ptrs) {
                int start = 0;
                for (int g = 0; g < groups; g++) {
                    size_t cnt = (size_t)(end[g] + 1 - start) * k;
                    if (prec[g]) CK(cudaMemcpy(M + (size_t)start * k, ptrs[g], sizeof(float) * cnt, cudaMemcpyDeviceToHost));
                    else {
                        std::vector<__half> h(cnt);
                        CK(cudaMemcpy(h.data(), ptrs[g], sizeof(__half) * cnt, cudaMemcpyDeviceToHost));
                        for (size_t j = 0; j < cnt; j++) M[(size_t)start * k + j] = __half2float(h[j]);
                    }
                    start = end[g] + 1;
                }
            };
            fetch(Pout.data(), uend, uprec, (int)ug, up); fetch(Qout.data(), iend, iprec, (int)ig, ip);
            std::vector<float> gp(ug * k), gq(ig * k), nsp(ug), nsq(ig);
            CK(cudaMemcpy(gp.data(), dGp, sizeof(float) * ug * k, cudaMemcpyDeviceToHost));
            CK(cudaMemcpy(gq.data(), dGq, sizeof(float) * ig * k, cudaMemcpyDeviceToHost));
            CK(cudaMemcpy(nsp.data(), dNp, sizeof(float) * ug, cudaMemcpyDeviceToHost));
            CK(cudaMemcpy(nsq.data(), dNq, sizeof(float) * ig, cudaMemcpyDeviceToHost));
            put(out, name + ".gsum_p", 0, gp.data(), ug * k); put(out, name + ".gsum_q", 0, gq.data(), ig * k);
            put(out, name + ".nsum_p", 0, nsp.data(), ug); put(out, name + ".nsum_q", 0, nsq.data(), ig);
            for (void* d : up) cudaFree(d);
            for (void* d : ip) cudaFree(d);
            if (k == 128) {
                // the "naive" variant (-v 6) on the same inputs and the same random sequence: it differs
                // from the kernel above only in how it looks a row's group up
                std::vector<void*> up2, ip2;
                build(P, uend, uprec, (int)ug, up2); build(Q, iend, iprec, (int)ig, ip2);
                void** dUp2 = to_dev(up2.data(), ug); void** dIp2 = to_dev(ip2.data(), ig);
                CK(cudaMemset(dGp, 0, sizeof(float) * ug * k)); CK(cudaMemset(dGq, 0, sizeof(float) * ig * k));
                seed_state<<<1, 1>>>(dState, seed);
                // this kernel reads its group ends from tables shifted by one entry, with -1 in front
                // (mf_methods.cu:1027-1046): entry g is the end of group g-1
                std::vector<unsigned int> ushift(ug + 1), ishift(ig + 1);
                ushift[0] = (unsigned int)-1; ishift[0] = (unsigned int)-1;
                for (uint64_t g = 0; g < ug; g++) ushift[g + 1] = uend[g];
                for (uint64_t g = 0; g < ig; g++) ishift[g + 1] = iend[g];
                unsigned int* dUshift = to_dev(ushift.data(), ug + 1); unsigned int* dIshift = to_dev(ishift.data(), ig + 1);
                naive_mascot_sgd_k128_hogwild_kernel<<<1, 32>>>(dR, nnz, dUp2, dIp2, dState, lr, k, update_count, vec, lam,
                    dUshift, dIshift, dUprec, dIprec, dGp, dGq, dNp, dNq, first_sample, (int)ug, (int)ig);
                CK(cudaDeviceSynchronize());
                std::vector<float> P2(np), Q2(nq);
                fetch(P2.data(), uend, uprec, (int)ug, up2); fetch(Q2.data(), iend, iprec, (int)ig, ip2);
                CK(cudaMemcpy(gp.data(), dGp, sizeof(float) * ug * k, cudaMemcpyDeviceToHost));
                CK(cudaMemcpy(gq.data(), dGq, sizeof(float) * ig * k, cudaMemcpyDeviceToHost));
                CK(cudaMemcpy(nsp.data(), dNp, sizeof(float) * ug, cudaMemcpyDeviceToHost));
                CK(cudaMemcpy(nsq.data(), dNq, sizeof(float) * ig, cudaMemcpyDeviceToHost));
                put(out, name + ".naive_P_out", 0, P2.data(), np); put(out, name + ".naive_Q_out", 0, Q2.data(), nq);
                put(out, name + ".naive_gsum_p", 0, gp.data(), ug * k); put(out, name + ".naive_gsum_q", 0, gq.data(), ig * k);
                put(out, name + ".naive_nsum_p", 0, nsp.data(), ug); put(out, name + ".naive_nsum_q", 0, nsq.data(), ig);
                for (void* d : up2) cudaFree(d);
                for (void* d : ip2) cudaFree(d);
            }
        } else if (kind == 7) {  // whole-model switching trainer (-v 8): binary16 (extra0 = 0) or fp32 (1)
            float *dSum, *dNorms;
            CK(cudaMalloc(&dSum, sizeof(float) * k)); CK(cudaMemset(dSum, 0, sizeof(float) * k));
            CK(cudaMalloc(&dNorms, sizeof(float))); CK(cudaMemset(dNorms, 0, sizeof(float)));
            const unsigned char cur_precision = (unsigned char)extra0;
            std::vector<__half> hp(np), hq(nq);
            void *dP, *dQ;
            if (!cur_precision) {
                for (size_t j = 0; j < np; j++) hp[j] = __float2half_rn(P[j]);
                for (size_t j = 0; j < nq; j++) hq[j] = __float2half_rn(Q[j]);
                dP = to_dev(hp.data(), np); dQ = to_dev(hq.data(), nq);
            } else {
                dP = to_dev(P, np); dQ = to_dev(Q, nq);
            }
            switching_only_sgd_k128_hogwild_kernel<<<1, 32>>>(dR, nnz, dP, dQ, dState, lr, k, update_count, vec, lam,
                                                               cur_precision, first_sample, dSum, dNorms);
            CK(cudaDeviceSynchronize());
            if (!cur_precision) {
                CK(cudaMemcpy(hp.data(), dP, sizeof(__half) * np, cudaMemcpyDeviceToHost));
                CK(cudaMemcpy(hq.data(), dQ, sizeof(__half) * nq, cudaMemcpyDeviceToHost));
                for (size_t j = 0; j < np; j++) Pout[j] = __half2float(hp[j]);
                for (size_t j = 0; j < nq; j++) Qout[j] = __half2float(hq[j]);
            } else {
                CK(cudaMemcpy(Pout.data(), dP, sizeof(float) * np, cudaMemcpyDeviceToHost));
                CK(cudaMemcpy(Qout.data(), dQ, sizeof(float) * nq, cudaMemcpyDeviceToHost));
            }
            std::vector<float> sv(k); float nrm;
            CK(cudaMemcpy(sv.data(), dSum, sizeof(float) * k, cudaMemcpyDeviceToHost));
            CK(cudaMemcpy(&nrm, dNorms, sizeof(float), cudaMemcpyDeviceToHost));
            put(out, name + ".sum_updated_val", 0, sv.data(), k);
            put(out, name + ".sum_norms", 0, &nrm, 1);
            cudaFree(dP); cudaFree(dQ); cudaFree(dSum); cudaFree(dNorms);
        } else if (kind == 3) {  // fp16 storage, fp32 arithmetic
            std::vector<__half> hp(np), hq(nq);
            for (size_t j = 0; j < np; j++) hp[j] = __float2half_rn(P[j]);
            for (size_t j = 0; j < nq; j++) hq[j] = __float2half_rn(Q[j]);
            __half* dP = to_dev(hp.data(), np); __half* dQ = to_dev(hq.data(), nq);
            if (k == 128) mem_quant_sgd_k128_hogwild_kernel<<<1, 32>>>(dR, nnz, dP, dQ, dState, lr, k, 1, 0, update_count, vec, lam);
            else mem_quant_sgd_k64_hogwild_kernel<<<1, 32>>>(dR, nnz, dP, dQ, dState, lr, k, 1, 0, update_count, vec, lam);
            CK(cudaDeviceSynchronize());
            CK(cudaMemcpy(hp.data(), dP, sizeof(__half) * np, cudaMemcpyDeviceToHost));
            CK(cudaMemcpy(hq.data(), dQ, sizeof(__half) * nq, cudaMemcpyDeviceToHost));
            for (size_t j = 0; j < np; j++) Pout[j] = __half2float(hp[j]);
            for (size_t j = 0; j < nq; j++) Qout[j] = __half2float(hq[j]);
            cudaFree(dP); cudaFree(dQ);
        } else {
            float* dP = to_dev(P, np); float* dQ = to_dev(Q, nq);
            if (kind == 0) {
                if (k == 128) single_sgd_k128_hogwild_kernel<<<1, 32>>>(dR, nnz, dP, dQ, dState, lr, k, update_count, vec, lam);
                else single_sgd_k64_hogwild_kernel<<<1, 32>>>(dR, nnz, dP, dQ, dState, lr, k, update_count, vec, lam);
            } else if (kind == 2) {
                float scaling = 1000;
                __half scaled_lambda = __float2half_rn(lam * scaling);
                if (k == 128) mpt_sgd_k128_hogwild_kernel<<<1, 32>>>(dR, nnz, dP, dQ, dState, lr, k, update_count, vec, scaled_lambda, scaling);
                else mpt_sgd_k64_hogwild_kernel<<<1, 32>>>(dR, nnz, dP, dQ, dState, lr, k, update_count, vec, scaled_lambda, scaling);
            } else if (kind == 4) {
                float *dSum, *dNorms;
                CK(cudaMalloc(&dSum, sizeof(float) * k)); CK(cudaMemset(dSum, 0, sizeof(float) * k));
                CK(cudaMalloc(&dNorms, sizeof(float)));
                unsigned char bits = (unsigned char)extra0;
                if (k == 128) muppet_sgd_k128_hogwild_kernel<<<1, 32>>>(dR, nnz, dP, dQ, dState, lr, k, update_count, vec, lam,
                                                                        first_sample, dSum, dNorms, bits, bits);
                else muppet_sgd_k64_hogwild_kernel<<<1, 32>>>(dR, nnz, dP, dQ, dState, lr, k, update_count, vec, lam,
                                                              first_sample, dSum, dNorms, bits, bits);
                CK(cudaDeviceSynchronize());
                std::vector<float> s(k); float nrm;
                CK(cudaMemcpy(s.data(), dSum, sizeof(float) * k, cudaMemcpyDeviceToHost));
                CK(cudaMemcpy(&nrm, dNorms, sizeof(float), cudaMemcpyDeviceToHost));
                put(out, name + ".sum_updated_val", 0, s.data(), k);
                put(out, name + ".sum_norms", 0, &nrm, 1);
                cudaFree(dSum); cudaFree(dNorms);
            } else if (kind == 5) {
                if (k == 128) afp_sgd_k128_hogwild_kernel<<<1, 32>>>(dR, nnz, dP, dQ, dState, lr, k, extra0, update_count, vec, lam);
                else afp_sgd_k64_hogwild_kernel<<<1, 32>>>(dR, nnz, dP, dQ, dState, lr, k, extra0, update_count, vec, lam);
            }
            CK(cudaDeviceSynchronize());
            CK(cudaMemcpy(Pout.data(), dP, sizeof(float) * np, cudaMemcpyDeviceToHost));
            CK(cudaMemcpy(Qout.data(), dQ, sizeof(float) * nq, cudaMemcpyDeviceToHost));
            cudaFree(dP); cudaFree(dQ);
        }
        CK(cudaGetLastError());
        put(out, name + ".P_out", 0, Pout.data(), np);
        put(out, name + ".Q_out", 0, Qout.data(), nq);
        cudaFree(dR); cudaFree(dState); cudaFree(dStarts);
    }
    write_bundle(argv[2], out);
    printf("wrote %s (%zu entries)\n", argv[2], out.size());
    return 0;
}
