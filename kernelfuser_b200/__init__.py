"""B200-native fused Q/K RMSNorm + RoPE + GQA attention (drop-in for
KernelFuser's ``optimized_attention``)."""
from .api import (KernelStatusError, attention_forward, attention_full, check_status, factored_attention,  # noqa: F401
                  fused, launch_attention,
                  optimized_attention, optimized_attention_host, optimized_attention_static,
                  prepare_rows, release_host_pipelines, selftest_wait_timeout, status_word)
from .inputs import WORKLOADS, Workload, make_inputs, make_workload_inputs, rope_tables  # noqa: F401

__all__ = ["optimized_attention", "optimized_attention_host", "optimized_attention_static", "factored_attention", "fused", "prepare_rows", "attention_forward", "attention_full", "launch_attention", "check_status",
           "status_word", "KernelStatusError", "selftest_wait_timeout", "release_host_pipelines", "make_inputs", "make_workload_inputs", "rope_tables",
           "WORKLOADS", "Workload"]
