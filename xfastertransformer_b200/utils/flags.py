"""Environment-flag registry (the reference's ``Env`` singleton, ``src/utils/environment.h:21-399``).

Hardware-neutral names are kept; Xeon-only ones (AMX thresholds, THP, NUMA weight
placement, oneCCL selection) are accepted and ignored so existing launch scripts run.
torchrun-style rank detection is added next to the MPI variables.
"""
from __future__ import annotations

import os
from typing import List


def _int(name: str, default: int) -> int:
    v = os.environ.get(name)
    if v is None or v == "":
        return default
    try:
        return int(v)
    except ValueError:
        return default


class Env:
    _inst = None

    def __init__(self):
        self.reload()

    @classmethod
    def get(cls) -> "Env":
        if cls._inst is None:
            cls._inst = cls()
        return cls._inst

    def reload(self) -> None:
        e = os.environ
        self.verbose = _int("XFT_VERBOSE", 0)
        self.pipeline_stage = max(1, _int("XFT_PIPELINE_STAGE", 1))
        self.max_request_num = max(1, _int("XFT_MAX_REQUEST_NUM", 1))
        self.flash_attn_threshold = _int("FLASH_ATTN_THRESHOLD", 8192)
        self.cat_mlp = _int("ENABLE_CAT_MLP", 1) != 0
        self.fake_model = _int("XFT_FAKE_MODEL", 0)      # 1: zeros (reference), 2: N(0,0.02) random
        self.fake_load_info = _int("XFT_FAKE_LOAD_INFO", 0) != 0
        self.debug_dir = e.get("XFT_DEBUG_DIR", "")
        wl = e.get("XFT_TIMELINE_WHITELIST", "")
        self.timeline_whitelist: List[str] = [s.strip() for s in wl.split(",") if s.strip()]
        self.timeline = _int("XFT_TIMELINE", 0) != 0
        self.single_instance = _int("SINGLE_INSTANCE", 0) != 0
        self.moe_engine = _int("XFT_MOE_ENGINE", 1)
        self.moe_split_balance_dim = _int("XFT_MOE_SPLIT_BALANCE_DIM", 0)
        self.engine = e.get("XFT_ENGINE", "")             # "", "CPU", "GPU[:idx]"
        # new flags of this build
        self.kv_block_size = _int("XFT_KV_BLOCK_SIZE", 64)
        self.cuda_graph = _int("XFT_CUDA_GRAPH", 1) != 0
        self.expert_parallel = _int("XFT_EXPERT_PARALLEL", 0) != 0
        self.fused_comm = _int("XFT_FUSED_COMM", 1) != 0
        # data-parallel attention + expert-parallel MoE: every rank keeps the whole attention stack and runs it on its
        # own share of the sequences; tokens travel to the ranks that own their experts and back (all-to-all)
        self.attention_dp = _int("XFT_ATTENTION_DP", 0) != 0
        self.moe_fused_a2a = _int("XFT_MOE_FUSED_A2A", 0) != 0      # with attention_dp: token exchange as peer-memory stores
        self.kv_cache_gb = float(e.get("XFT_KV_CACHE_GB", "0") or 0)
        self.prefix_cache = _int("XFT_PREFIX_CACHE", 0) != 0      # reuse the KV blocks of prompts that share a prefix
        # greedy decoding with n-gram drafts: up to this many tokens are copied from an earlier occurrence of the current
        # suffix and checked in ONE forward; accepted ones cost no extra step (output identical to plain greedy)
        self.spec_ngram = max(0, _int("XFT_SPEC_NGRAM", 0))
        self.max_batch_tokens = _int("XFT_MAX_BATCH_TOKENS", 8192)
        self.step_timeout_s = float(e.get("XFT_STEP_TIMEOUT_S", "0") or 0)
        self.fuse_norm = _int("XFT_FUSE_NORM", 1) != 0    # fold RMSNorm gains into the consuming bf16 GEMM
        self.attn_tma = _int("XFT_ATTN_TMA", 1) != 0      # bf16 decode attention through the TMA ring kernel
        self.attn_splits = _int("XFT_ATTN_SPLITS", 0)     # decode split-KV factor; 0 = planned per launch
        self.gemm_persistent = _int("XFT_GEMM_PERSISTENT", 0) != 0     # prefill GEMMs through the persistent kernel
        # prompt-size bf16 GEMMs (more than 128 tokens) through the persistent token-major kernel
        self.gemm_prefill_tm = _int("XFT_GEMM_PREFILL_TM", 1) != 0
        self.gemm_prefill_tm_all = _int("XFT_GEMM_PREFILL_TM", 1) == 2     # 2: also gated and long-K products
        # decode-size bf16 GEMMs (up to 64 tokens) through the balanced weight-stream kernel (gemm_decode_sm100.cu);
        # XFT_FUSE_QKV_ROPE: RoPE + cache append as the epilogue of the QKV product (head_dim 128, bf16 cache)
        # prompt attention through the tcgen05 kernel from this many query rows on (head_dim 128, bf16 cache, no ALiBi);
        # a very large value switches it off
        self.attn_tc_min_q = _int("XFT_ATTN_TC_MIN_Q", 2)
        self.gemm_streamk = _int("XFT_GEMM_STREAMK", 1) != 0
        self.fuse_qkv_rope = _int("XFT_FUSE_QKV_ROPE", 1) != 0
        # tensor-parallel prefill: two groups of prompts are interleaved block by block, so that the all-reduce of one
        # overlaps the compute of the other
        self.prefill_overlap = _int("XFT_PREFILL_OVERLAP", 0) != 0
        # XFT_PREFILL_FUSED_AR (row-parallel prefill GEMM + all-reduce as one kernel) and XFT_MAX_BATCH_TOKENS size the
        # symmetric buffers: parallel/fused_comm.py reads them when the peer communicator is built
        # accepted, no effect on a GPU build
        self.ignored = {k: e.get(k) for k in (
            "XFT_USE_AMX_M", "ENABLE_TUNED_COMM", "ENABLE_KV_TRANS", "ENABLE_THP", "XFT_ONECCL",
            "XFT_PRIMITIVE_CACHE_M", "FIRST_TOKEN_WEIGHT_LOCATION", "NEXT_TOKEN_WEIGHT_LOCATION") if k in e}

    @staticmethod
    def launched_multi_rank() -> bool:
        """True under mpirun (``messenger.h:228-233``) or torchrun."""
        e = os.environ
        if _int("SINGLE_INSTANCE", 0):
            return False
        mpi = any(k in e for k in ("MPI_LOCALRANKID", "MPI_LOCALNRANKS", "PMI_RANK", "PMI_SIZE", "PMIX_RANK",
                                   "OMPI_COMM_WORLD_RANK"))
        return mpi or (_int("WORLD_SIZE", 1) > 1 and "RANK" in e)
