// Retrieval-quality scorer of the eval-retrieval command on the accelerated path.
// Restates computeRetrievalQuality / topRetrievalScores and the metric helpers of the reference
// (runtime/retrieval_eval.go:541-726 of odvcencio/manta) around ONE change: the per-query scan of all documents with
// a bounded heap (:586-616) becomes fused score + top-k passes on the device over the documents bound once.  The
// reference orders equal scores by document ID string (:618-626); the device orders equal scores by row index, so the
// documents are bound in ID order and the two rules coincide.
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <numeric>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../../include/manta_b200_host.h"
#include "half.h"
#include "json.h"

namespace {

int fail(char** err, const char* fmt, ...) {
    if (err) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        size_t n = strlen(buf) + 1;
        char* out = (char*)malloc(n);
        if (out) memcpy(out, buf, n);
        *err = out;
    }
    return 1;
}

using Rels = std::unordered_map<std::string, double>;

// idealDCGAt, retrieval_eval.go:681-701
double ideal_dcg_at(const Rels& rels, int k) {
    std::vector<double> values;
    for (const auto& kv : rels)
        if (kv.second > 0) values.push_back(kv.second);
    std::sort(values.begin(), values.end(), [](double a, double b) { return a > b; });
    double dcg = 0.0;
    const int limit = std::min<int>(k, (int)values.size());
    for (int i = 0; i < limit; ++i) dcg += values[i] / std::log2((double)i + 2.0);
    return dcg;
}

double rel_of(const Rels& rels, const std::string& id) {
    auto it = rels.find(id);
    return it == rels.end() ? 0.0 : it->second;
}

}  // namespace

extern "C" int manta_b200_retrieval_quality(MantaB200Runtime* rt, const float* query_vectors, const char* const* query_ids,
                                            int n_queries, const float* doc_vectors, const char* const* doc_ids, int64_t n_docs,
                                            int dim, const char* const* qrel_query_ids, const char* const* qrel_doc_ids,
                                            const double* qrel_values, int64_t n_qrels, int top_k, char** out_json, char** err) {
    if (!rt || !out_json) return fail(err, "retrieval_quality: NULL argument");
    *out_json = nullptr;
    if (n_queries < 0 || n_docs <= 0 || dim <= 0) return fail(err, "retrieval_quality: bad shape (%d queries, %lld docs, dim %d)", n_queries, (long long)n_docs, dim);
    if ((n_queries > 0 && (!query_vectors || !query_ids)) || !doc_vectors || !doc_ids) return fail(err, "retrieval_quality: NULL argument");
    if (n_qrels > 0 && (!qrel_query_ids || !qrel_doc_ids || !qrel_values)) return fail(err, "retrieval_quality: NULL qrels");
    if (top_k < 100) top_k = 100;                                   // :546-548
    const int k = (int)std::min<int64_t>(top_k, n_docs);           // topRetrievalScores clamps to the corpus, :587-589
    if (k > 1024) return fail(err, "retrieval_quality: top_k %d exceeds the fused pass maximum 1024", k);

    // documents in ID order (stable, so that duplicate IDs keep their input order)
    std::vector<int64_t> order((size_t)n_docs);
    std::iota(order.begin(), order.end(), (int64_t)0);
    std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return strcmp(doc_ids[a], doc_ids[b]) < 0; });
    std::unordered_map<std::string, bool> doc_set;
    doc_set.reserve((size_t)n_docs * 2);
    for (int64_t i = 0; i < n_docs; ++i) doc_set[doc_ids[i]] = true;
    std::vector<uint16_t> bits((size_t)n_docs * dim);
    for (int64_t r = 0; r < n_docs; ++r) {
        const float* src = doc_vectors + (size_t)order[(size_t)r] * dim;
        for (int c = 0; c < dim; ++c) bits[(size_t)r * dim + c] = mb200_host::half_bits(src[c]);
    }
    MantaB200Candidates* set = nullptr;
    if (manta_b200_candidates_bind(rt, MANTA_B200_LAYOUT_F16, n_docs, dim, bits.data(), nullptr, 0, MANTA_B200_MEM_HOST, &set, err)) return 1;
    std::vector<uint16_t>().swap(bits);

    // qrels[query][doc] = relevance (later lines of a file overwrite earlier ones, as map assignment does)
    std::unordered_map<std::string, Rels> qrels;
    for (int64_t i = 0; i < n_qrels; ++i) qrels[qrel_query_ids[i]][qrel_doc_ids[i]] = qrel_values[i];

    // queries that have at least one relevant document in the corpus (:555-570)
    struct Eval {
        int query;
        Rels rels;
    };
    std::vector<Eval> evals;
    int64_t relevant_pairs = 0, skipped_relevant_docs = 0, skipped_no_relevant = 0;
    for (int q = 0; q < n_queries; ++q) {
        Eval e;
        e.query = q;
        auto it = qrels.find(query_ids[q]);
        if (it != qrels.end())
            for (const auto& kv : it->second) {
                if (doc_set.count(kv.first)) e.rels[kv.first] = kv.second;
                else ++skipped_relevant_docs;
            }
        if (e.rels.empty()) {
            ++skipped_no_relevant;
            continue;
        }
        relevant_pairs += (int64_t)e.rels.size();
        evals.push_back(std::move(e));
    }

    double ndcg10 = 0.0, mrr10 = 0.0, recall10 = 0.0, recall100 = 0.0;
    const int kBatch = 256;
    std::vector<uint16_t> qbits;
    std::vector<int32_t> ids;
    std::vector<float> scores;
    int rc = 0;
    for (size_t b0 = 0; b0 < evals.size() && !rc; b0 += kBatch) {
        const int nb = (int)std::min<size_t>(kBatch, evals.size() - b0);
        qbits.assign((size_t)nb * dim, 0);
        for (int i = 0; i < nb; ++i) {
            const float* src = query_vectors + (size_t)evals[b0 + i].query * dim;
            for (int c = 0; c < dim; ++c) qbits[(size_t)i * dim + c] = mb200_host::half_bits(src[c]);
        }
        ids.resize((size_t)nb * k);
        scores.resize((size_t)nb * k);
        rc = manta_b200_score_topk(rt, set, MANTA_B200_METRIC_DOT, MANTA_B200_ORDER_LARGEST, qbits.data(), nb, k, ids.data(), scores.data(), err);
        if (rc) break;
        for (int i = 0; i < nb; ++i) {
            const Rels& rels = evals[b0 + i].rels;
            const int32_t* row = ids.data() + (size_t)i * k;
            auto id_at = [&](int j) { return std::string(doc_ids[order[(size_t)row[j]]]); };
            // ndcgAt :663-679, mrrAt :703-711, recallAt :713-725
            double dcg = 0.0;
            const int l10 = std::min(10, k), l100 = std::min(100, k);
            for (int j = 0; j < l10; ++j) {
                const double rel = rel_of(rels, id_at(j));
                if (rel > 0) dcg += rel / std::log2((double)j + 2.0);
            }
            const double idcg = ideal_dcg_at(rels, 10);
            ndcg10 += (idcg == 0) ? 0.0 : dcg / idcg;
            for (int j = 0; j < l10; ++j)
                if (rel_of(rels, id_at(j)) > 0) {
                    mrr10 += 1.0 / (double)(j + 1);
                    break;
                }
            int h10 = 0, h100 = 0;
            for (int j = 0; j < l100; ++j)
                if (rel_of(rels, id_at(j)) > 0) {
                    if (j < l10) ++h10;
                    ++h100;
                }
            recall10 += (double)h10 / (double)rels.size();
            recall100 += (double)h100 / (double)rels.size();
        }
    }
    char* uerr = nullptr;
    manta_b200_candidates_unbind(rt, set, &uerr);
    free(uerr);
    if (rc) return 1;
    const double denom = evals.empty() ? 1.0 : (double)evals.size();
    using mjson::Value;
    Value root = Value::make_object();
    Value quality = Value::make_object();
    auto num = [](double v) {
        Value x;
        x.kind = Value::Number;
        x.num = v;
        return x;
    };
    quality.set("ndcg_at_10", num(ndcg10 / denom));
    quality.set("mrr_at_10", num(mrr10 / denom));
    quality.set("recall_at_10", num(recall10 / denom));
    quality.set("recall_at_100", num(recall100 / denom));
    root.set("quality", quality);
    root.set("evaluated_queries", num((double)evals.size()));
    root.set("relevant_pairs", num((double)relevant_pairs));
    root.set("skipped_relevant_docs", num((double)skipped_relevant_docs));
    root.set("skipped_no_relevant", num((double)skipped_no_relevant));
    root.set("scored_pairs", num((double)evals.size() * (double)n_docs));  // :167
    root.set("top_k", num((double)k));
    std::string text;
    mjson::write(root, &text);
    char* out = (char*)malloc(text.size() + 1);
    if (!out) return fail(err, "retrieval_quality: out of memory");
    memcpy(out, text.c_str(), text.size() + 1);
    *out_json = out;
    return 0;
}
