// rbm.hpp -- row-block-merged (RBM) view of an ELLPACK matrix, built on the host at load time.
// Same plan as the reference's build_rbm_from_ellpack (include/rbm_conv.hpp:8-31,
// src/layers/rbm_conv.cpp:7-73): rows are grouped in blocks of Ct_max; per block the union of
// column ids (ascending) with, per union column, the (row-in-block, weight) pairs in ascending
// row order.  Per row the pairs appear in ascending column order, so a kernel consuming the plan
// keeps every row's accumulation chain unchanged.
#pragma once

#include <cstdint>
#include <vector>

#include "ellpack.hpp"

namespace spx {

struct RBMColPair {
    uint16_t row;   ///< row id within the block [0, Ct)
    float w;
};

struct RBMBlock {
    uint32_t M0 = 0;                 ///< first row of the block
    uint32_t Ct = 0;                 ///< rows in the block (<= Ct_max)
    std::vector<uint32_t> krel;      ///< union column ids, ascending
    std::vector<uint32_t> colptr;    ///< krel.size()+1 offsets into pairs
    std::vector<RBMColPair> pairs;
    std::vector<float> bias;         ///< Ct values, empty without bias
};

struct RBMPlan {
    uint32_t M = 0, N = 0, Ct_max = 0;
    std::vector<RBMBlock> blocks;
};

RBMPlan build_rbm_from_ellpack(const Ellpack& E, const float* bias_or_null, uint32_t Ct_max = 8);

}  // namespace spx

#ifndef SPX_NO_GLOBAL_NAMES
using spx::RBMBlock;
using spx::RBMColPair;
using spx::RBMPlan;
using spx::build_rbm_from_ellpack;
#endif
