"""bench.py's host side: the contract of its command line and of the record it prints, without a GPU."""
import json
import os
import subprocess
import sys

import helpers

sys.path.insert(0, helpers.ROOT)
import bench  # noqa: E402


def test_more_than_one_gpu_is_refused_with_one_line():
    proc = subprocess.run([sys.executable, os.path.join(helpers.ROOT, "bench.py"), "--gpus", "2"], capture_output=True,
                          text=True, timeout=120)
    assert proc.returncode == 2
    assert proc.stdout.strip().count("\n") == 0 and "one GPU" in proc.stdout


def test_reference_arm_says_why_it_cannot_run_here():
    """Without a GPU the reference arm prints its `unavailable` line with the reason and exits 0."""
    proc = subprocess.run([sys.executable, os.path.join(helpers.ROOT, "bench.py"), "--impl", "reference"],
                          capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "no CUDA device" in line["unavailable"]


def test_config_is_flat_and_names_every_size():
    class Args:
        batch, steps = 8, 256
    cfg = bench.workload_config(Args, 16, {"source": "measured"})
    assert len(cfg) <= 20 and all(not isinstance(v, (dict, list)) for v in cfg.values())
    for key in ("layers", "layers_full", "hidden_size", "heads", "kv_heads", "head_dim", "intermediate_size",
                "vocab_size", "global_batch", "seq_len", "prompt_len", "new_tokens", "prefill_tokens"):
        assert key in cfg, key
    assert cfg["layers"] == cfg["layers_full"] == 16 and cfg["seq_len"] == 4096


def test_flop_count_of_the_prompt_step():
    """The 1B shape at 2,048 tokens: 3.99 TFLOP of products (the head on the last row only) and 0.275 TFLOP of
    causal attention."""
    total = bench.prefill_flops(bench.CONFIG_1B, 16, [2048])
    d, ff = 2048, 8192
    per_token = 2 * (d * 3072 + 2048 * d + 3 * d * ff)
    assert abs(16 * per_token * 2048 / 1e12 - 3.986) < 0.01
    assert abs(total / 1e12 - 4.26) < 0.01
    two = bench.prefill_flops(bench.CONFIG_1B, 16, [1024, 1024])
    assert two < total                      # two short prompts attend to less than one long one


def test_kernel_table_fractions():
    rows = [{"stage": "FFN", "kernel": "k1", "launches": 32, "us": 2000.0, "bytes": 2.0e9, "flops": 4.0e12},
            {"stage": "", "kernel": "k2", "launches": 2, "us": 100.0, "bytes": 0.0, "flops": 0.0}]
    text = bench.kernel_table(rows, 2, {"hbm_gbs": 5000.0, "bf16_tflops": 2000.0}, "title")
    lines = text.splitlines()
    assert lines[0] == "### title" and "| FFN | k1 | 16 | 1000.0 | 95.2 % | 1000.00 | 1000 | 20.0 % | 2000.00 | 2000.0 | 100.0 % |" in text
    assert lines[-1].startswith("| | **sum** | 17 | 1050.0 |")


def test_shapes_of_the_benchmark_set():
    assert bench.CONFIG_3B["num_hidden_layers"] == 28 and bench.CONFIG_3B["head_dim"] == 128
    assert bench.CONFIG_8B["intermediate_size"] == 14336 and bench.CONFIG_8B["tie_word_embeddings"] is False
    assert bench.CONFIG_8B["rope_scaling"]["factor"] == 8.0 and bench.CONFIG_1B["rope_scaling"]["factor"] == 32.0
    from llm_infer_engine_b200.config import load_config
    for cfg in (bench.CONFIG_1B, bench.CONFIG_3B, bench.CONFIG_8B):
        arch, typed = load_config(cfg)
        assert arch.name == "LlamaForCausalLM" and typed.vocab_size == 128256
