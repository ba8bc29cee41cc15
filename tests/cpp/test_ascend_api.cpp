// Exercises the faiss::ascend classes the way the reference's own unit tests do
// (FR/ut/cases/flat/TestAscendFlat.cpp:76-88, FR/ut/cases/int8_flat/TestAscendInt8Flat.cpp:87-103,
//  FR/ut/TestAscendIndexUTIVFPQ.cpp:77-183, FR/ut/cases/multi_search/TestAscendIndexUTMultiSearchFlat.cpp:94-118):
// constructor / parameter rejection with exact message substrings, ntotal bookkeeping,
// copyFrom / copyTo round trips, reset, remove -- plus, in "gpu" mode, numerical checks against
// a brute-force scan written in this file.
//   usage: test_ascend_api cpu|gpu
#include <faiss/ascend/AscendIndexFlat.h>
#include <faiss/ascend/AscendIndexIVFPQ.h>
#include <faiss/ascend/AscendIndexInt8Flat.h>
#include <faiss/ascend/AscendCloner.h>
#include <faiss/ascend/AscendMultiIndexSearch.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <memory>
#include <random>
#include <string>
#include <vector>

using namespace faiss;
using namespace faiss::ascend;

static int g_fail = 0, g_checks = 0;
#define CHECK(cond)                                                        \
    do {                                                                   \
        ++g_checks;                                                        \
        if (!(cond)) {                                                     \
            ++g_fail;                                                      \
            std::printf("FAIL %s:%d  %s\n", __FILE__, __LINE__, #cond);   \
        }                                                                  \
    } while (0)

static bool throws_with(const std::function<void()>& f, const char* needle) {
    try {
        f();
    } catch (const FaissException& e) {
        if (std::strstr(e.what(), needle)) return true;
        std::printf("  message was: %s\n", e.what());
        return false;
    } catch (...) {
        return false;
    }
    return false;
}

static std::vector<float> gauss(size_t n, int d, unsigned seed) {
    std::mt19937 rng(seed);
    std::normal_distribution<float> nd(0.f, 1.f);
    std::vector<float> v(n * d);
    for (auto& x : v) x = nd(rng);
    return v;
}

static void test_parameter_errors() {
    CHECK(throws_with([] { AscendIndexFlat ix(100, METRIC_L2); }, "Invalid number of dimensions(100), should be divisible by 16"));
    CHECK(throws_with([] { AscendIndexFlat ix(48, METRIC_L2); }, "Unsupported dims"));
    CHECK(throws_with([] { AscendIndexFlat ix(5000 * 16, METRIC_L2); }, "Invalid number of dimensions"));
    CHECK(throws_with([] { AscendIndexFlat ix(128, static_cast<MetricType>(5)); }, "Unsupported metric type"));
    CHECK(throws_with([] { AscendIndexFlat ix(128, METRIC_L2, AscendIndexFlatConfig({0, 0})); }, "some device IDs are the same"));
    CHECK(throws_with([] { AscendIndexFlat ix(128, METRIC_L2, AscendIndexFlatConfig(std::vector<int>{})); }, "device list should be in range"));
    CHECK(throws_with([] { AscendIndexFlat ix(128, METRIC_L2, AscendIndexFlatConfig({0}, -5)); }, "should be -1 or in range [0, 10240MB]!"));
    CHECK(throws_with([] { AscendIndexFlat ix(static_cast<const IndexFlat*>(nullptr)); }, "Invalid index nullptr."));
    CHECK(throws_with([] { AscendIndexInt8Flat ix(100, METRIC_L2); }, "should be divisible by 16"));
    CHECK(throws_with([] { AscendIndexInt8Flat ix(32, METRIC_L2); }, "Unsupported dims 32"));
    CHECK(throws_with([] { AscendIndexInt8Flat ix(64, METRIC_L2, AscendIndexInt8FlatConfig(1000)); }, "Unsupported blockSize 1000"));
    CHECK(throws_with([] { AscendIndexIVFPQ ix(128, METRIC_INNER_PRODUCT, 1024, 16, 8); }, "Unsupported metric type"));
    CHECK(throws_with([] { AscendIndexIVFPQ ix(64, METRIC_L2, 1024, 16, 8); }, "Unsupported dims: 64"));
    CHECK(throws_with([] { AscendIndexIVFPQ ix(128, METRIC_L2, 1000, 16, 8); }, "Unsupported nlists: 1000"));
    CHECK(throws_with([] { AscendIndexIVFPQ ix(128, METRIC_L2, 1024, 3, 8); }, "Unsupported msubs: 3"));
    CHECK(throws_with([] { AscendIndexIVFPQ ix(128, METRIC_L2, 1024, 16, 4); }, "Unsupported nbits: 4"));
    // config defaults the reference documents
    AscendIndexConfig c;
    CHECK(c.deviceList == std::vector<int>{0} && c.resourceSize == 0x2000000 && c.dBlockSize == 262144 && !c.slim);
    AscendIndexFlatConfig fc;
    CHECK(fc.resourceSize == INDEX_DEFAULT_MEM);
    AscendIndexIVFPQConfig pc;
    CHECK(pc.cp.niter == 10 && pc.trainSamplesPerList == 40 && pc.maxTrainSamples == 10000000 && pc.pqNiter == -1 &&
          !pc.useKmeansPP && !pc.enableQueryParallelSearch && pc.resourceSize == IVF_DEFAULT_MEM);
    std::vector<AscendIndex*> none;
    float D[1];
    idx_t I[1];
    float x[128] = {0};
    CHECK(throws_with([&] { Search(none, 1, x, 1, D, I, true); }, "size of indexes (0) must be > 0 and <= 10000."));
}

static void test_no_gpu_failure() {
    // valid parameters, no device: construction must fail loudly, not fall back to a CPU path
    CHECK(throws_with([] { AscendIndexFlat ix(128, METRIC_L2); }, "create index failed"));
    CHECK(throws_with([] { AscendIndexInt8Flat ix(64, METRIC_INNER_PRODUCT); }, "create index failed"));
}

static void brute(const std::vector<float>& xb, const std::vector<float>& xq, int d, bool l2, int k,
                  const std::vector<idx_t>& ids, std::vector<float>& D, std::vector<idx_t>& I) {
    const size_t nb = xb.size() / d, nq = xq.size() / d;
    D.assign(nq * k, 0.f);
    I.assign(nq * k, -1);
    for (size_t q = 0; q < nq; ++q) {
        std::vector<std::pair<double, size_t>> all(nb);
        for (size_t i = 0; i < nb; ++i) {
            double acc = 0;
            for (int t = 0; t < d; ++t) {
                const double a = xq[q * d + t], b = xb[i * d + t];
                acc += l2 ? (a - b) * (a - b) : a * b;
            }
            all[i] = {l2 ? acc : -acc, i};
        }
        std::partial_sort(all.begin(), all.begin() + k, all.end());
        for (int j = 0; j < k; ++j) {
            D[q * k + j] = static_cast<float>(l2 ? all[j].first : -all[j].first);
            I[q * k + j] = ids.empty() ? static_cast<idx_t>(all[j].second) : ids[all[j].second];
        }
    }
}

static std::vector<float> round_half(const std::vector<float>& v) {
    std::vector<float> o(v.size());
    for (size_t i = 0; i < v.size(); ++i) o[i] = static_cast<float>(static_cast<_Float16>(v[i]));
    return o;
}

static void test_flat_gpu() {
    const int d = 128, k = 10;
    const size_t nb = 20000, nq = 17;
    auto xb = gauss(nb, d, 1), xq = gauss(nq, d, 2);
    for (MetricType metric : {METRIC_L2, METRIC_INNER_PRODUCT}) {
        AscendIndexFlat ix(d, metric);
        CHECK(ix.ntotal == 0 && ix.is_trained && ix.d == d && ix.getDeviceList() == std::vector<int>{0});
        ix.add(static_cast<idx_t>(nb / 2), xb.data());
        ix.add(static_cast<idx_t>(nb - nb / 2), xb.data() + (nb / 2) * d);
        CHECK(ix.ntotal == static_cast<idx_t>(nb) && ix.getBaseSize(0) == nb);
        std::vector<float> D(nq * k), Dr;
        std::vector<idx_t> I(nq * k), Ir;
        ix.search(static_cast<idx_t>(nq), xq.data(), k, D.data(), I.data());
        brute(round_half(xb), round_half(xq), d, metric == METRIC_L2, k, {}, Dr, Ir);   // fp16 storage, as the reference
        size_t same = 0;
        double maxrel = 0;
        for (size_t i = 0; i < D.size(); ++i) {
            same += I[i] == Ir[i];
            maxrel = std::max(maxrel, std::fabs(D[i] - Dr[i]) / std::max(1e-6, static_cast<double>(std::fabs(Dr[i]))));
        }
        CHECK(same >= D.size() - 2);          // a near-tie may swap two neighbours
        CHECK(maxrel < 1e-3);
        // self hit at rank 1 (FR/test/ascend/TestAscendIndexFlat.cpp:117-123)
        if (metric == METRIC_L2) {
            ix.search(5, xb.data(), 1, D.data(), I.data());
            for (int q = 0; q < 5; ++q) CHECK(I[q] == q);
        }
        CHECK(throws_with([&] { ix.search(0, xq.data(), k, D.data(), I.data()); }, "n must be > 0 and < 1000000000"));
        CHECK(throws_with([&] { ix.search(1, xq.data(), 5000, D.data(), I.data()); }, "k must be > 0 and <= 4096"));
        CHECK(throws_with([&] { ix.search(1, static_cast<const float*>(nullptr), k, D.data(), I.data()); }, "x cannot be nullptr."));
        CHECK(throws_with([&] { ix.search(1, xq.data(), k, nullptr, I.data()); }, "distance cannot be nullptr."));
        CHECK(throws_with([&] { ix.search(1, xq.data(), k, D.data(), nullptr); }, "labels cannot be nullptr."));
        // copyTo / copyFrom round trip keeps results
        IndexFlat cpu(d, metric);
        ix.copyTo(&cpu);
        CHECK(cpu.ntotal == static_cast<idx_t>(nb) && cpu.codes.size() == nb * d * sizeof(float));
        AscendIndexFlat ix2(&cpu);
        std::vector<float> D2(nq * k);
        std::vector<idx_t> I2(nq * k);
        ix.search(static_cast<idx_t>(nq), xq.data(), k, D.data(), I.data());
        ix2.search(static_cast<idx_t>(nq), xq.data(), k, D2.data(), I2.data());
        CHECK(I == I2 && D == D2);
        // search_with_masks: only rows whose bit is set may appear (every third row kept); the
        // fp16-query overload answers like the float one on fp16-rounded queries
        {
            const size_t mrow = (nb + 7) / 8;
            std::vector<uint8_t> mask(nq * mrow, 0);
            for (size_t q = 0; q < nq; ++q)
                for (size_t i = q % 3; i < nb; i += 3) mask[q * mrow + i / 8] |= static_cast<uint8_t>(1u << (i % 8));
            std::vector<float> Dm(nq * k), Dh(nq * k);
            std::vector<idx_t> Im(nq * k), Ih(nq * k);
            ix.search_with_masks(static_cast<idx_t>(nq), xq.data(), k, Dm.data(), Im.data(), mask.data());
            bool kept_only = true, sorted = true;
            for (size_t q = 0; q < nq; ++q)
                for (int j = 0; j < k; ++j) {
                    kept_only = kept_only && Im[q * k + j] >= 0 && static_cast<size_t>(Im[q * k + j]) % 3 == q % 3;
                    if (j) sorted = sorted && (metric == METRIC_L2 ? Dm[q * k + j - 1] <= Dm[q * k + j]
                                                                 : Dm[q * k + j - 1] >= Dm[q * k + j]);
                }
            CHECK(kept_only && sorted);
            std::vector<uint16_t> xh(nq * d);
            for (size_t i = 0; i < xh.size(); ++i) {
                const _Float16 hv = static_cast<_Float16>(xq[i]);
                std::memcpy(&xh[i], &hv, 2);
            }
            ix.search_with_masks(static_cast<idx_t>(nq), xh.data(), k, Dh.data(), Ih.data(), mask.data());
            CHECK(Ih == Im && Dh == Dm);
            CHECK(throws_with([&] { ix.search_with_masks(1, xq.data(), k, Dm.data(), Im.data(), nullptr); }, "mask can not be nullptr."));
        }
        // remove + reset
        IDSelectorRange sel(0, 100);
        CHECK(ix.remove_ids(sel) == 100 && ix.ntotal == static_cast<idx_t>(nb - 100));
        ix.search(static_cast<idx_t>(nq), xq.data(), k, D.data(), I.data());
        for (idx_t id : I) CHECK(id >= 100);
        ix.reset();
        CHECK(ix.ntotal == 0 && ix.getBaseSize(0) == 0);
    }
    // ids through IndexIDMap
    IndexFlat sub(d, METRIC_L2);
    IndexIDMap idmap(&sub);
    std::vector<idx_t> ids(1000);
    for (size_t i = 0; i < ids.size(); ++i) ids[i] = 5000 + 3 * static_cast<idx_t>(i);
    idmap.add_with_ids(1000, xb.data(), ids.data());
    AscendIndexFlat ix(&idmap);
    std::vector<float> D(5);
    std::vector<idx_t> I(5);
    ix.search(5, xb.data(), 1, D.data(), I.data());
    for (int q = 0; q < 5; ++q) CHECK(I[q] == ids[q]);
    std::vector<idx_t> map;
    ix.getIdxMap(0, map);
    CHECK(map == ids);
}

static void test_int8_gpu() {
    const int d = 64, k = 8;
    const size_t nb = 9000, nq = 6;
    std::mt19937 rng(3);
    std::vector<int8_t> xb(nb * d), xq(nq * d);
    for (auto& v : xb) v = static_cast<int8_t>(static_cast<int>(rng() % 256) - 128);
    for (auto& v : xq) v = static_cast<int8_t>(static_cast<int>(rng() % 256) - 128);
    AscendIndexInt8Flat ix(d, METRIC_INNER_PRODUCT);
    ix.add(static_cast<idx_t>(nb), xb.data());
    CHECK(ix.getNTotal() == static_cast<idx_t>(nb) && ix.getDim() == d && ix.isTrained());
    std::vector<float> D(nq * k);
    std::vector<idx_t> I(nq * k);
    ix.search(static_cast<idx_t>(nq), xq.data(), k, D.data(), I.data());
    for (size_t q = 0; q < nq; ++q) {
        std::vector<std::pair<int64_t, size_t>> all(nb);
        for (size_t i = 0; i < nb; ++i) {
            int64_t acc = 0;
            for (int t = 0; t < d; ++t) acc += static_cast<int>(xq[q * d + t]) * static_cast<int>(xb[i * d + t]);
            all[i] = {-acc, i};
        }
        std::sort(all.begin(), all.end());
        for (int j = 0; j < k; ++j) {
            CHECK(I[q * k + j] == static_cast<idx_t>(all[j].second));
            CHECK(D[q * k + j] == static_cast<float>(-all[j].first));
        }
    }
    std::vector<int8_t> base;
    ix.getBase(0, base);
    CHECK(base == xb);
    IndexScalarQuantizer sq(d, ScalarQuantizer::QT_8bit, METRIC_INNER_PRODUCT);
    ix.copyTo(&sq);
    CHECK(sq.ntotal == static_cast<idx_t>(nb) && sq.codes.size() == nb * d);
    AscendIndexInt8Flat ix2(&sq);
    std::vector<float> D2(nq * k);
    std::vector<idx_t> I2(nq * k);
    ix2.search(static_cast<idx_t>(nq), xq.data(), k, D2.data(), I2.data());
    CHECK(I == I2 && D == D2);
    ix.reset();
    CHECK(ix.getNTotal() == 0);

    // the reference's own meaning of METRIC_INNER_PRODUCT on this index (fp16 cosine), behind the switch
    SetInt8InnerProductAsCosine(true);
    {
        AscendIndexInt8Flat cs(d, METRIC_INNER_PRODUCT);
        cs.add(static_cast<idx_t>(nb), xb.data());
        std::vector<int8_t> q2(xb.begin() + 17 * d, xb.begin() + 19 * d);   // two base rows as queries
        std::vector<float> Dc(2 * k);
        std::vector<idx_t> Ic(2 * k);
        cs.search(2, q2.data(), k, Dc.data(), Ic.data());
        for (int q = 0; q < 2; ++q) {
            bool found = false;
            for (int j = 0; j < k; ++j) {
                CHECK(Dc[q * k + j] <= 1.01f && Dc[q * k + j] >= -1.01f);
                if (j) CHECK(Dc[q * k + j] <= Dc[q * k + j - 1]);
                found = found || Ic[q * k + j] == 17 + q;
            }
            CHECK(found && Dc[q * k] > 0.99f);
        }
    }
    SetInt8InnerProductAsCosine(false);
    CHECK(!Int8InnerProductAsCosine());
}

static std::vector<float> mixture(size_t n, int d, int ncenters, unsigned seed, unsigned cseed) {
    auto cen = gauss(static_cast<size_t>(ncenters), d, cseed);
    std::mt19937 rng(seed);
    std::normal_distribution<float> nd(0.f, 0.1f);
    std::vector<float> v(n * d);
    for (size_t i = 0; i < n; ++i) {
        const size_t c = rng() % static_cast<unsigned>(ncenters);
        for (int t = 0; t < d; ++t) v[i * d + t] = cen[c * d + t] + nd(rng);
    }
    return v;
}

static void test_ivfpq_gpu() {
    const int d = 128, nlist = 1024, M = 16;
    const size_t nb = 40000, nq = 50;
    auto xb = mixture(nb, d, 256, 4, 99);
    AscendIndexIVFPQ ix(d, METRIC_L2, nlist, M, 8);
    CHECK(!ix.is_trained && ix.getNumLists() == nlist);
    std::vector<float> D(nq * 10);
    std::vector<idx_t> I(nq * 10);
    CHECK(throws_with([&] { ix.add(10, xb.data()); }, "Index not trained"));
    ix.train(static_cast<idx_t>(nb), xb.data());
    CHECK(ix.is_trained);
    std::vector<idx_t> ids(nb);
    for (size_t i = 0; i < nb; ++i) ids[i] = 7 + 2 * static_cast<idx_t>(i);
    ix.add_with_ids(static_cast<idx_t>(nb), xb.data(), ids.data());
    CHECK(ix.ntotal == static_cast<idx_t>(nb));
    uint32_t total = 0;
    for (int l = 0; l < nlist; ++l) total += ix.getListLength(l);
    CHECK(total == nb);
    CHECK(throws_with([&] { ix.setNumProbes(0); }, "nprobe must be greater than 0"));
    CHECK(throws_with([&] { ix.setNumProbes(nlist + 1); }, "nprobe must be less than or equal to nlist"));
    ix.setNumProbes(32);
    CHECK(ix.getNumProbes() == 32);
    // own id within the top 10 for (nearly) every base vector used as a query
    // (FR/test/ascend/TestAscendIndexIVFPQ.cpp:151-166 asserts the self hit)
    ix.search(static_cast<idx_t>(nq), xb.data(), 10, D.data(), I.data());
    size_t hit = 0;
    for (size_t q = 0; q < nq; ++q)
        for (int j = 0; j < 10; ++j) hit += I[q * 10 + j] == ids[q];
    CHECK(hit >= nq * 8 / 10);
    CHECK(throws_with([&] { ix.search(1, xb.data(), 321, D.data(), I.data()); }, "k must be > 0 and <= 320"));
    // reset + re-add gives byte-identical lists (TestAscendIndexIVFPQ.cpp:118-146)
    std::vector<uint8_t> c0, c1;
    std::vector<ascend_idx_t> i0, i1;
    int probe_list = 0;
    for (int l = 0; l < nlist; ++l)
        if (ix.getListLength(l) > 3) { probe_list = l; break; }
    ix.getListCodesAndIds(probe_list, c0, i0);
    CHECK(c0.size() == i0.size() * M && !i0.empty());
    ix.reset();
    CHECK(ix.ntotal == 0 && ix.is_trained && ix.getListLength(probe_list) == 0);
    ix.add_with_ids(static_cast<idx_t>(nb), xb.data(), ids.data());
    ix.getListCodesAndIds(probe_list, c1, i1);
    CHECK(c0 == c1 && i0 == i1);
    // copyTo / copyFrom round trip: same lists, same results
    std::vector<float> D1(nq * 10);
    std::vector<idx_t> I1(nq * 10);
    ix.search(static_cast<idx_t>(nq), xb.data(), 10, D1.data(), I1.data());
    IndexFlatL2 quant(d);
    IndexIVFPQ cpu(&quant, d, nlist, M, 8);
    ix.copyTo(&cpu);
    CHECK(cpu.ntotal == static_cast<idx_t>(nb) && !cpu.by_residual && cpu.quantizer->ntotal == nlist);
    AscendIndexIVFPQ ix2(d, METRIC_L2, nlist, M, 8);
    ix2.copyFrom(&cpu);
    CHECK(ix2.ntotal == static_cast<idx_t>(nb) && ix2.is_trained && ix2.getNumProbes() == 32);
    ix2.search(static_cast<idx_t>(nq), xb.data(), 10, D.data(), I.data());
    CHECK(D == D1 && I == I1);
    // remove by ids
    idx_t gone[2] = {ids[0], ids[1]};
    ix2.remove_ids(2, gone);
    CHECK(ix2.ntotal == static_cast<idx_t>(nb - 2));
}

static void test_multi_search_gpu() {
    const int d = 64, k = 5;
    const size_t nq = 9;
    auto xq = gauss(nq, d, 20);
    std::vector<std::vector<float>> bases;
    std::vector<std::unique_ptr<AscendIndexFlat>> owners;
    std::vector<AscendIndex*> idx;
    idx_t next = 0;
    for (int s = 0; s < 3; ++s) {
        const size_t n = 2000 + 500 * s;
        bases.push_back(gauss(n, d, 30 + s));
        owners.emplace_back(new AscendIndexFlat(d, METRIC_L2));
        std::vector<idx_t> ids(n);
        for (size_t i = 0; i < n; ++i) ids[i] = next++;
        owners.back()->add_with_ids(static_cast<idx_t>(n), bases.back().data(), ids.data());
        idx.push_back(owners.back().get());
    }
    std::vector<float> D(3 * nq * k), Dm(nq * k);
    std::vector<idx_t> I(3 * nq * k), Im(nq * k);
    Search(idx, static_cast<idx_t>(nq), xq.data(), k, D.data(), I.data(), false);   // [index][n][k]
    for (int s = 0; s < 3; ++s) {
        std::vector<float> Ds(nq * k);
        std::vector<idx_t> Is(nq * k);
        idx[s]->search(static_cast<idx_t>(nq), xq.data(), k, Ds.data(), Is.data());
        CHECK(std::equal(Ds.begin(), Ds.end(), D.begin() + s * nq * k));
        CHECK(std::equal(Is.begin(), Is.end(), I.begin() + s * nq * k));
    }
    Search(idx, static_cast<idx_t>(nq), xq.data(), k, Dm.data(), Im.data(), true);
    for (size_t q = 0; q < nq; ++q) {
        std::vector<std::pair<float, idx_t>> all;
        for (int s = 0; s < 3; ++s)
            for (int j = 0; j < k; ++j) all.push_back({D[(s * nq + q) * k + j], I[(s * nq + q) * k + j]});
        std::sort(all.begin(), all.end());
        for (int j = 0; j < k; ++j) CHECK(Dm[q * k + j] == all[j].first && Im[q * k + j] == all[j].second);
    }
    std::vector<float> big(1025 * d, 0.f);
    std::vector<float> Db(1025 * k);
    std::vector<idx_t> Ib(1025 * k);
    CHECK(throws_with([&] { Search(idx, 1025, big.data(), k, Db.data(), Ib.data(), true); }, "n must be > 0 and <= 1024"));
    CHECK(throws_with([&] { Search(idx, 1, xq.data(), 1025, Db.data(), Ib.data(), true); }, "k must be > 0 and <= 1024"));
    SetRelaxedLimits(true);
    Search(idx, 1025, big.data(), k, Db.data(), Ib.data(), true);   // relaxed: pages internally
    SetRelaxedLimits(false);
}

// index_cpu_to_ascend / index_ascend_to_cpu (FR/ascend/AscendCloner.cpp:64-99,159-196,232-281): a CPU
// index goes to the device and back with its vectors, ids and (IVFPQ) lists intact, and the device
// copy answers like an index built directly.
static void test_cloner_gpu() {
    const int d = 64;
    const size_t nb = 3000, nq = 7;
    auto xb = gauss(nb, d, 41);
    auto xq = gauss(nq, d, 42);
    // Flat behind an id map
    IndexFlat* cpu_flat = new IndexFlat(d, METRIC_L2);
    IndexIDMap cpu_map(cpu_flat);
    cpu_map.own_fields = true;
    std::vector<idx_t> ids(nb);
    for (size_t i = 0; i < nb; ++i) ids[i] = 1000 + 3 * static_cast<idx_t>(i);
    cpu_map.add_with_ids(static_cast<idx_t>(nb), xb.data(), ids.data());
    std::unique_ptr<faiss::Index> dev(index_cpu_to_ascend({0}, &cpu_map));
    CHECK(dynamic_cast<AscendIndexFlat*>(dev.get()) != nullptr && dev->ntotal == static_cast<idx_t>(nb));
    std::vector<float> D(nq * 5), D2(nq * 5);
    std::vector<idx_t> I(nq * 5), I2(nq * 5);
    dev->search(static_cast<idx_t>(nq), xq.data(), 5, D.data(), I.data());
    AscendIndexFlat direct(d, METRIC_L2);
    direct.add_with_ids(static_cast<idx_t>(nb), xb.data(), ids.data());
    direct.search(static_cast<idx_t>(nq), xq.data(), 5, D2.data(), I2.data());
    CHECK(D == D2 && I == I2);
    std::unique_ptr<faiss::Index> back(index_ascend_to_cpu(dev.get()));
    IndexIDMap* back_map = dynamic_cast<IndexIDMap*>(back.get());
    CHECK(back_map != nullptr && back_map->ntotal == static_cast<idx_t>(nb) && back_map->id_map == ids);
    CHECK(throws_with([&] { index_ascend_to_cpu(&cpu_map); }, "not supported for this type of Index"));
    CHECK(throws_with([&] { index_cpu_to_ascend({0}, &direct); }, "not supported for this type of Index"));
    // IVFPQ: device index -> CPU struct -> device index, identical lists and answers
    const int nlist = 1024, M = 16, d2 = 128;
    auto xv = mixture(20000, d2, 128, 4, 77);
    AscendIndexIVFPQ ix(d2, METRIC_L2, nlist, M, 8);
    ix.train(20000, xv.data());
    ix.add(20000, xv.data());
    ix.setNumProbes(16);
    std::unique_ptr<faiss::Index> cpu_pq(index_ascend_to_cpu(&ix));
    IndexIVFPQ* pq = dynamic_cast<IndexIVFPQ*>(cpu_pq.get());
    CHECK(pq != nullptr && pq->ntotal == 20000 && pq->nlist == static_cast<size_t>(nlist) && pq->pq.M == static_cast<size_t>(M));
    std::unique_ptr<faiss::Index> dev_pq(index_cpu_to_ascend(std::vector<int>{0}, pq));
    AscendIndexIVFPQ* ix2 = dynamic_cast<AscendIndexIVFPQ*>(dev_pq.get());
    CHECK(ix2 != nullptr && ix2->ntotal == 20000 && ix2->getNumProbes() == 16);
    std::vector<float> Da(nq * 10), Db(nq * 10);
    std::vector<idx_t> Ia(nq * 10), Ib(nq * 10);
    ix.search(static_cast<idx_t>(nq), xv.data(), 10, Da.data(), Ia.data());
    if (ix2) ix2->search(static_cast<idx_t>(nq), xv.data(), 10, Db.data(), Ib.data());
    CHECK(Da == Db && Ia == Ib);
    // int8: the index that is not a faiss::Index
    std::vector<int8_t> xi(2000 * 64);
    std::mt19937 rng(5);
    for (auto& v : xi) v = static_cast<int8_t>(static_cast<int>(rng() % 256) - 128);
    AscendIndexInt8Flat i8(64, METRIC_L2);
    i8.add(2000, xi.data());
    std::unique_ptr<faiss::Index> cpu8(index_int8_ascend_to_cpu(&i8));
    CHECK(cpu8 != nullptr && cpu8->ntotal == 2000);
    std::unique_ptr<AscendIndexInt8> dev8(index_int8_cpu_to_ascend({0}, cpu8.get()));
    CHECK(dev8 != nullptr && dev8->getNTotal() == 2000);
    std::vector<float> D8a(3 * 4), D8b(3 * 4);
    std::vector<idx_t> I8a(3 * 4), I8b(3 * 4);
    i8.search(3, xi.data(), 4, D8a.data(), I8a.data());
    if (dev8) dev8->search(3, xi.data(), 4, D8b.data(), I8b.data());
    CHECK(D8a == D8b && I8a == I8b);
}

// Two devices (skipped on a box with one): an index spread over both answers fp16 queries, and the
// query-parallel IVFPQ layout (enableQueryParallelSearch: the index replicated, the queries split)
// answers exactly like the index on one device.
static void test_two_devices_gpu(int ndev) {
    if (ndev < 2) {
        std::printf("two-device checks skipped (%d device)\n", ndev);
        return;
    }
    const int d = 64;
    const size_t nb = 5000, nq = 11;
    auto xb = gauss(nb, d, 51);
    auto xq = gauss(nq, d, 52);
    AscendIndexFlatConfig two({0, 1});
    AscendIndexFlat spread(d, METRIC_L2, two), one(d, METRIC_L2);
    spread.add(static_cast<idx_t>(nb), xb.data());
    one.add(static_cast<idx_t>(nb), xb.data());
    std::vector<uint16_t> xh(nq * d);
    for (size_t i = 0; i < xh.size(); ++i) {
        const _Float16 h = static_cast<_Float16>(xq[i]);
        std::memcpy(&xh[i], &h, 2);
    }
    std::vector<float> D(nq * 5), D1(nq * 5);
    std::vector<idx_t> I(nq * 5), I1(nq * 5);
    spread.search(static_cast<idx_t>(nq), xh.data(), 5, D.data(), I.data());
    one.search(static_cast<idx_t>(nq), xh.data(), 5, D1.data(), I1.data());
    CHECK(D == D1 && I == I1);
    const int nlist = 1024, M = 16, d2 = 128;
    auto xv = mixture(20000, d2, 128, 4, 78);
    AscendIndexIVFPQConfig rc({0, 1});
    rc.enableQueryParallelSearch = true;
    AscendIndexIVFPQ rep(d2, METRIC_L2, nlist, M, 8, rc), single(d2, METRIC_L2, nlist, M, 8);
    rep.train(20000, xv.data());
    single.train(20000, xv.data());
    rep.add(20000, xv.data());
    single.add(20000, xv.data());
    CHECK(rep.ntotal == 20000);
    uint32_t total = 0;
    for (int l = 0; l < nlist; ++l) total += rep.getListLength(l);
    CHECK(total == 20000);
    rep.setNumProbes(16);
    single.setNumProbes(16);
    const size_t nq2 = 37;
    std::vector<float> Da(nq2 * 10), Db(nq2 * 10);
    std::vector<idx_t> Ia(nq2 * 10), Ib(nq2 * 10);
    rep.search(static_cast<idx_t>(nq2), xv.data(), 10, Da.data(), Ia.data());
    single.search(static_cast<idx_t>(nq2), xv.data(), 10, Db.data(), Ib.data());
    CHECK(Da == Db && Ia == Ib);
}

int main(int argc, char** argv) {
    const std::string mode = argc > 1 ? argv[1] : "cpu";
    test_parameter_errors();
    if (mode == "cpu") {
        test_no_gpu_failure();
    } else {
        test_flat_gpu();
        test_int8_gpu();
        test_ivfpq_gpu();
        test_multi_search_gpu();
        test_cloner_gpu();
        test_two_devices_gpu(argc > 2 ? std::atoi(argv[2]) : 1);
    }
    std::printf("%d checks, %d failed\n", g_checks, g_fail);
    return g_fail ? 1 : 0;
}
