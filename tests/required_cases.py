"""Required cases: tests whose skip or expected-failure must never pass silently.

A run in which one of these was collected but ended as skipped, xfailed or xpassed-under-a-non-strict-mark is turned into
a failing run by ``conftest.py`` (the reference's ``scripts/check-required-cases.py`` does the same for its result files:
a skipped required case is a failed gate, not a green one).  Entries are node-id prefixes.  ``GPU`` entries are enforced
only when a CUDA device is present (without one every GPU test is skipped by design).
"""

CPU = [
    "tests/test_oracle_tiny_llama.py",
    "tests/test_engine_emulated.py",
    "tests/test_tp_emulated.py",
    "tests/test_failure_cpu.py",
    "tests/test_lifecycle.py",
    "tests/test_planner.py",
    "tests/test_serve.py",
    "tests/test_driver.py",
]

GPU = [
    "tests/test_kernels_gpu.py::test_gemm_tcgen05",
    "tests/test_kernels_gpu.py::test_gemm_skinny",
    "tests/test_kernels_gpu.py::test_attn_paged",
    "tests/test_kernels_gpu.py::test_flash_prefill_matches_reference_over_paged_kv",
    "tests/test_kernels_gpu.py::test_rope_kv_write",
    "tests/test_kernels_gpu.py::test_rmsnorm",
    "tests/test_kernels_gpu.py::test_argmax",
    "tests/test_engine_gpu.py::test_prefill_logits_match_reference",
    "tests/test_engine_gpu.py::test_decode_steps_equal_prefill",
    "tests/test_engine_gpu.py::test_chained_decode_matches_stepwise",
    "tests/test_quant_gpu.py::test_quant_gemv_matches_dequantised_reference",
    "tests/test_moe_gpu.py::test_mixtral_like_model_matches_reference",
    "tests/test_driver_gpu.py::test_generate_with_chunked_prefill_matches_reference",
    "tests/test_failure_gpu.py::test_peer_flag_wait_runs_out_and_is_reported",
    "tests/test_zz_no_alloc.py::test_noalloc_attention_matches_regular_entry_point_twice",
]
