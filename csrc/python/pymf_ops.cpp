// `ops` submodule: raw launchers of the fused compute+collective kernels. Arguments are device addresses (ints) and a
// CUDA stream handle; the torch-facing wrappers live in memfabric_hybrid_b200/ops.
#include <pybind11/stl.h>

#include <cuda_runtime.h>

#include "../kernels/mf_kernels.h"
#include "pymf_parts.h"

namespace py = pybind11;

void BindOps(py::module_ &m)
{
    py::module_ ops = m.def_submodule("ops", "raw launchers of the fused kernels");

    ops.attr("AR_AUTO") = (int)MF_AR_AUTO;
    ops.attr("AR_ONESHOT") = (int)MF_AR_ONESHOT;
    ops.attr("AR_TWOSHOT") = (int)MF_AR_TWOSHOT;
    ops.attr("AR_NVLS") = (int)MF_AR_NVLS;
    ops.attr("AR_ONESHOT_NOTAIL") = (int)MF_AR_ONESHOT_NOTAIL;
    ops.attr("ALLREDUCE_ARGS_BYTES") = (int)sizeof(mf_allreduce_args_t);

    // Packs one argument block (to be copied to device memory by the caller).
    ops.def("pack_allreduce_args", [](uint64_t meta, uint64_t x, uint64_t residual, uint64_t weight, uint64_t residualOut, uint64_t out, uint64_t status,
                                       uint64_t epochState) {
        mf_allreduce_args_t a{};
        a.meta = (const void *)meta;
        a.x = (const void *)x;
        a.residual = (const void *)residual;
        a.weight = (const void *)weight;
        a.residualOut = (void *)residualOut;
        a.out = (void *)out;
        a.status = (int *)status;
        a.epochState = (unsigned long long *)epochState;
        return py::bytes((const char *)&a, sizeof(a));
    }, py::arg("meta"), py::arg("x"), py::arg("residual"), py::arg("weight"), py::arg("residual_out"), py::arg("out"), py::arg("status"),
       py::arg("epoch_state") = 0);
    ops.attr("GEMM_EPI_BF16") = (int)MF_GEMM_EPI_BF16;
    ops.attr("GEMM_EPI_SWIGLU") = (int)MF_GEMM_EPI_SWIGLU;
    ops.attr("GEMM_EPI_SWIGLU_FP8") = (int)MF_GEMM_EPI_SWIGLU_FP8;
    ops.attr("MOE_MAX_SIBLINGS") = (int)MF_MOE_MAX_SIBLINGS;
    ops.def("moe_grouped_gemm_mx", [](uint64_t a, uint64_t aSf, uint64_t b, uint64_t bScale, uint64_t out, uint64_t outSf, uint64_t groupOffset,
                                      uint64_t groupCount, int G, int rowsTotal, int N, int K, int mode, int tileN, uint64_t status, int ctas,
                                      uint64_t stream, uint64_t arrive, uint64_t waitNs) {
        if (arrive != 0) {
            return mf_k_moe_grouped_gemm_mx_gated((const void *)a, (const uint32_t *)aSf, (const void *)b, (const float *)bScale, (void *)out,
                                                  (void *)outSf, (const int *)groupOffset, (const int *)groupCount, G, rowsTotal, N, K, mode, tileN,
                                                  (const int *)arrive, waitNs, (int *)status, ctas, (mf_stream_t)stream);
        }
        return mf_k_moe_grouped_gemm_mx((const void *)a, (const uint32_t *)aSf, (const void *)b, (const float *)bScale, (void *)out, (void *)outSf,
                                        (const int *)groupOffset, (const int *)groupCount, G, rowsTotal, N, K, mode, tileN, (int *)status, ctas,
                                        (mf_stream_t)stream);
    }, py::arg("a"), py::arg("a_sf"), py::arg("b"), py::arg("b_scale"), py::arg("out"), py::arg("out_sf"), py::arg("group_offset"),
            py::arg("group_count"), py::arg("G"), py::arg("rows_total"), py::arg("N"), py::arg("K"), py::arg("mode"), py::arg("tile_n") = 0,
            py::arg("status") = 0, py::arg("ctas") = 0, py::arg("stream") = 0, py::arg("arrive") = 0, py::arg("wait_ns") = 0);
    ops.attr("GEMM_B_PACKED") = (int)MF_GEMM_B_PACKED;
    ops.attr("GEMM_ARRIVAL_EXPIRED") = (int)MF_K_GEMM_ARRIVAL_EXPIRED;
    ops.attr("GEMM_PIPELINE_EXPIRED") = (int)MF_K_GEMM_PIPELINE_EXPIRED;
    ops.def("moe_grouped_gemm", [](uint64_t a, uint64_t aScale, uint64_t b, uint64_t bScale, uint64_t out, uint64_t groupOffset, uint64_t groupCount,
                                   int G, int rowsTotal, int N, int K, int mode, uint64_t status, int ctas, uint64_t stream) {
        return mf_k_moe_grouped_gemm((const void *)a, (const float *)aScale, (const void *)b, (const float *)bScale, (void *)out,
                                     (const int *)groupOffset, (const int *)groupCount, G, rowsTotal, N, K, mode, (int *)status, ctas, (mf_stream_t)stream);
    }, py::arg("a"), py::arg("a_scale"), py::arg("b"), py::arg("b_scale"), py::arg("out"), py::arg("group_offset"), py::arg("group_count"), py::arg("G"),
            py::arg("rows_total"), py::arg("N"), py::arg("K"), py::arg("mode"), py::arg("status") = 0, py::arg("ctas") = 0, py::arg("stream") = 0);
    ops.def("quant_rows_fp8", [](uint64_t x, uint64_t q, uint64_t scale, int rows, int K, uint64_t rowLimit, uint64_t stream) {
        return mf_k_quant_rows_fp8((const void *)x, (void *)q, (float *)scale, rows, K, (const int *)rowLimit, (mf_stream_t)stream);
    }, py::arg("x"), py::arg("q"), py::arg("scale"), py::arg("rows"), py::arg("K"), py::arg("row_limit") = 0, py::arg("stream") = 0);
    ops.attr("MOE_DISPATCH_ARGS_BYTES") = (int)sizeof(mf_moe_dispatch_args_t);
    ops.attr("MOE_COMBINE_ARGS_BYTES") = (int)sizeof(mf_moe_combine_args_t);
    ops.def("pack_moe_dispatch_args", [](uint64_t meta, uint64_t x, uint64_t topkIdx, uint64_t topkW, uint64_t cnt, uint64_t recvX, uint64_t recvSf,
                                         uint64_t recvMeta, uint64_t recvSib, uint64_t localCnt, uint64_t cursor, uint64_t expertOffset, uint64_t expertCount,
                                         uint64_t sendSlot, uint64_t status, int T, int cap, uint64_t arrive, int dedupMinPairs, uint64_t epochState) {
        mf_moe_dispatch_args_t a{};
        a.arrive = (int *)arrive;
        a.dedupMinPairs = dedupMinPairs;
        a.epochState = (unsigned long long *)epochState;
        a.meta = (const void *)meta;
        a.x = (const void *)x;
        a.topkIdx = (const int *)topkIdx;
        a.topkW = (const float *)topkW;
        a.cnt = (int *)cnt;
        a.recvX = (void *)recvX;
        a.recvSf = (uint32_t *)recvSf;
        a.recvMeta = (int4 *)recvMeta;
        a.recvSib = (int2 *)recvSib;
        a.localCnt = (int *)localCnt;
        a.cursor = (int *)cursor;
        a.expertOffset = (int *)expertOffset;
        a.expertCount = (int *)expertCount;
        a.sendSlot = (int *)sendSlot;
        a.status = (int *)status;
        a.T = T;
        a.cap = cap;
        return py::bytes((const char *)&a, sizeof(a));
    }, py::arg("meta"), py::arg("x"), py::arg("topk_idx"), py::arg("topk_w"), py::arg("cnt"), py::arg("recv_x"), py::arg("recv_sf"), py::arg("recv_meta"),
            py::arg("recv_sib"), py::arg("local_cnt"), py::arg("cursor"), py::arg("expert_offset"), py::arg("expert_count"), py::arg("send_slot"),
            py::arg("status"), py::arg("T"), py::arg("cap"), py::arg("arrive") = 0, py::arg("dedup_min_pairs") = 0, py::arg("epoch_state") = 0);
    ops.def("pack_moe_combine_args", [](uint64_t meta, uint64_t y, uint64_t recvMeta, uint64_t recvSib, uint64_t expertOffset, uint64_t expertCount,
                                        uint64_t retY, uint64_t topkIdx, uint64_t out, uint64_t status, int T, int cap, int retRows, uint64_t epochState) {
        mf_moe_combine_args_t a{};
        a.epochState = (unsigned long long *)epochState;
        a.meta = (const void *)meta;
        a.y = (const void *)y;
        a.recvMeta = (const int4 *)recvMeta;
        a.recvSib = (const int2 *)recvSib;
        a.expertOffset = (const int *)expertOffset;
        a.expertCount = (const int *)expertCount;
        a.retY = (void *)retY;
        a.topkIdx = (const int *)topkIdx;
        a.out = (void *)out;
        a.status = (int *)status;
        a.T = T;
        a.cap = cap;
        a.retRows = retRows;
        return py::bytes((const char *)&a, sizeof(a));
    }, py::arg("meta"), py::arg("y"), py::arg("recv_meta"), py::arg("recv_sib"), py::arg("expert_offset"), py::arg("expert_count"), py::arg("ret_y"),
            py::arg("topk_idx"), py::arg("out"), py::arg("status"), py::arg("T"), py::arg("cap"), py::arg("ret_rows"), py::arg("epoch_state") = 0);
    ops.def("moe_dispatch", [](uint64_t argsDev, int nEmulated, int rankCount, int H, int K, int E, uint32_t channel, uint64_t epoch, uint64_t timeoutNs,
                               int ctas, uint64_t stream) {
        return mf_k_moe_dispatch((const mf_moe_dispatch_args_t *)argsDev, nEmulated, rankCount, H, K, E, channel, epoch, timeoutNs, ctas,
                                 (mf_stream_t)stream);
    }, py::arg("args_dev"), py::arg("n_emulated"), py::arg("rank_count"), py::arg("H"), py::arg("K"), py::arg("E"), py::arg("channel"), py::arg("epoch"),
            py::arg("timeout_ns") = 0, py::arg("ctas") = 0, py::arg("stream") = 0);
    ops.def("moe_combine", [](uint64_t argsDev, int nEmulated, int rankCount, int H, int K, int EL, uint32_t channel, uint64_t epoch, uint64_t timeoutNs,
                              int ctas, uint64_t stream) {
        return mf_k_moe_combine((const mf_moe_combine_args_t *)argsDev, nEmulated, rankCount, H, K, EL, channel, epoch, timeoutNs, ctas,
                                (mf_stream_t)stream);
    }, py::arg("args_dev"), py::arg("n_emulated"), py::arg("rank_count"), py::arg("H"), py::arg("K"), py::arg("EL"), py::arg("channel"), py::arg("epoch"),
            py::arg("timeout_ns") = 0, py::arg("ctas") = 0, py::arg("stream") = 0);
    ops.attr("RESHARD_DESC_BYTES") = (int)sizeof(mf_reshard_desc_t);
    ops.attr("RESHARD_ARGS_BYTES") = (int)sizeof(mf_reshard_args_t);
    ops.def("pack_reshard_desc", [](uint64_t srcFlatOff, uint64_t dstOff, uint64_t scaleOff, uint32_t colsFull, uint32_t r0, uint32_t c0, uint32_t nrows,
                                    uint32_t ncols, uint32_t tileStart, uint32_t quant) {
        mf_reshard_desc_t d{srcFlatOff, dstOff, scaleOff, colsFull, r0, c0, nrows, ncols, tileStart, quant, 0};
        return py::bytes((const char *)&d, sizeof(d));
    });
    ops.def("pack_reshard_args", [](uint64_t meta, uint64_t srcShard, uint64_t dst, uint64_t dstScale, uint64_t descs, uint64_t status, uint64_t shardElems,
                                    uint32_t ndesc, uint32_t totalTiles) {
        mf_reshard_args_t a{};
        a.meta = (const void *)meta;
        a.srcShard = (const void *)srcShard;
        a.dst = (void *)dst;
        a.dstScale = (float *)dstScale;
        a.descs = (const mf_reshard_desc_t *)descs;
        a.status = (int *)status;
        a.shardElems = shardElems;
        a.ndesc = ndesc;
        a.totalTiles = totalTiles;
        return py::bytes((const char *)&a, sizeof(a));
    });
    ops.def("reshard", [](uint64_t argsDev, int nEmulated, int rankCount, uint32_t channel, uint64_t epoch, uint64_t timeoutNs, int ctas, uint64_t stream) {
        return mf_k_reshard((const mf_reshard_args_t *)argsDev, nEmulated, rankCount, channel, epoch, timeoutNs, ctas, (mf_stream_t)stream);
    }, py::arg("args_dev"), py::arg("n_emulated"), py::arg("rank_count"), py::arg("channel"), py::arg("epoch"), py::arg("timeout_ns") = 0,
            py::arg("ctas") = 0, py::arg("stream") = 0);
    ops.def("allreduce_rmsnorm", [](uint64_t argsDev, int nEmulated, int rankCount, int T, int H, float eps, int algo, uint32_t channel, uint64_t epoch,
                                    uint64_t timeoutNs, int ctas, uint64_t stream) {
        return mf_k_allreduce_rmsnorm((const mf_allreduce_args_t *)argsDev, nEmulated, rankCount, T, H, eps, algo, channel, epoch, timeoutNs, ctas,
                                      (mf_stream_t)stream);
    }, py::arg("args_dev"), py::arg("n_emulated"), py::arg("rank_count"), py::arg("T"), py::arg("H"), py::arg("eps"), py::arg("algo"),
            py::arg("channel"), py::arg("epoch"), py::arg("timeout_ns") = 0, py::arg("ctas") = 0, py::arg("stream") = 0);
}
