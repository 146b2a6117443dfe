"""Quality and routing experiments that run on this engine's own model (PyTorch path, any device): stale tensor
parallelism, confidence-adaptive top-k routing, route predictability, self-speculation depth curve, greedy-output
quality gates, numerical check of the block-fp8 weights, and the HTML report of a context sweep.

The reference runs the same experiments as monkey patches of a vLLM install (experiments/stale_tp/stale_tp.py,
experiments/adaptive_topk/vllm_adaptive_moe.py) and as stand-alone scripts over HF models (tools/router_mass.py,
tools/routing_predict.py, tools/verify_route_prediction.py, tools/verify_self_speculation.py,
tools/quality_probe.py, tools/quality_compare.py, tools/validate_fp8_quant.py, tools/gen_report.py); here they use
the hooks of ``models.qwen3_moe.Qwen3MoE`` (``route_fn``, the collectives object) directly.
"""
