// rbm.cpp -- see rbm.hpp.  Rows of a block are already sorted by column, so the union is built
// with a Ct-way merge (one cursor per row) instead of sorting all triples.
#include "rbm.hpp"

#include <algorithm>
#include <limits>

namespace spx {

RBMPlan build_rbm_from_ellpack(const Ellpack& E, const float* bias_or_null, uint32_t Ct_max)
{
    if (Ct_max == 0 || Ct_max > 65535) throw std::runtime_error("build_rbm_from_ellpack: Ct_max out of range");
    RBMPlan P;
    P.M = E.m;
    P.N = E.n;
    P.Ct_max = Ct_max;
    for (uint32_t M0 = 0; M0 < E.m; M0 += Ct_max) {
        RBMBlock B;
        B.M0 = M0;
        B.Ct = std::min(Ct_max, E.m - M0);
        B.colptr.push_back(0);
        std::vector<uint32_t> cur(B.Ct, 0);
        for (;;) {
            // smallest column id any row of the block still has to emit
            uint32_t k = std::numeric_limits<uint32_t>::max();
            bool any = false;
            for (uint32_t t = 0; t < B.Ct; ++t) {
                const uint32_t i = M0 + t;
                if (cur[t] < E.nnz[i]) {
                    k = std::min(k, E.idx[size_t(i) * E.r + cur[t]]);
                    any = true;
                }
            }
            if (!any) break;
            B.krel.push_back(k);
            for (uint32_t t = 0; t < B.Ct; ++t) {
                const uint32_t i = M0 + t;
                if (cur[t] < E.nnz[i] && E.idx[size_t(i) * E.r + cur[t]] == k) {
                    B.pairs.push_back(RBMColPair{ uint16_t(t), E.Wd.ptr[size_t(i) * E.r + cur[t]] });
                    ++cur[t];
                }
            }
            B.colptr.push_back(uint32_t(B.pairs.size()));
        }
        if (bias_or_null) B.bias.assign(bias_or_null + M0, bias_or_null + M0 + B.Ct);
        P.blocks.push_back(std::move(B));
    }
    return P;
}

}  // namespace spx
