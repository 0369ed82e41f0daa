"""B200-native fault-tolerant FP8 GEMM (ABFT) behind the C-ABI of include/ft_gemm.h."""
from ._abi import (FT_ABFT_TILE, FT_ERR_CUDA, FT_ERR_INVALID, FT_ERR_TIMEOUT, FT_ERR_UNSUPPORTED, FT_MAX_FAULTS,
                   FT_MAX_RECORDS, FT_OK, FtGemmError, LIB_PATH, load)
from .attention import FAULT_NONE, FAULT_OUTPUT, FAULT_SCORE, FAULT_SOFTMAX, FAULT_SOFTMAX_STATE, AttnReport, FtAttention, gather_attention_reports, shard_heads
from .gemm_softmax import GemmSoftmaxAbft, GsReport, generate_gs_fp8
from .operator import AbftGemm, HostAbftGemm, Report, TileRecord, generate_fp8
from .sharding import RowShard, gather_reports, shard_rows

__all__ = ["GemmSoftmaxAbft", "GsReport", "generate_gs_fp8", "FtAttention", "AttnReport", "shard_heads", "gather_attention_reports", "FAULT_NONE", "FAULT_SCORE", "FAULT_SOFTMAX", "FAULT_SOFTMAX_STATE", "FAULT_OUTPUT", "AbftGemm", "HostAbftGemm", "Report", "TileRecord", "generate_fp8", "RowShard", "shard_rows",
           "gather_reports", "load", "LIB_PATH", "FtGemmError", "FT_OK", "FT_ERR_INVALID", "FT_ERR_CUDA",
           "FT_ERR_TIMEOUT", "FT_ERR_UNSUPPORTED", "FT_ABFT_TILE", "FT_MAX_FAULTS", "FT_MAX_RECORDS"]
