"""One arm of a vLLM engine run on random ("dummy") weights: the drop-in protocol end to end.

    python -m lcgemm.integrate.engine_run --arm optimized --tokens 2048 [--layers 64]

What the reference's harness does with a real checkpoint (``lcgemm/bench/prefill.py:76-176``),
minus the checkpoint: ``arm()`` before the engine exists, an in-process vLLM engine built from
a hand-written Qwen3.5-style text config (hidden 5120, intermediate 17408, the 3 : 1
linear / full attention pattern) with ``load_format="dummy"``, ``install(llm, tokens)``, batch-1
prefills of exactly ``tokens`` token ids with one generated token, cold L2 before every timed
pass, and ``check_calls`` to prove every layer of every pass took the rank-7 chain and none the
functional branch.  ``--arm stock`` runs the same engine unpatched (in a process that never
imported the patch).  ``--layers`` below 64 shortens the model (the patch checks the count it is
told to expect); the result says so.  Prints one ``RESULT_JSON`` line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import tempfile
import time
from pathlib import Path

os.environ["VLLM_DISABLE_COMPILE_CACHE"] = "1"
os.environ["VLLM_ENABLE_V1_MULTIPROCESSING"] = "0"     # in-process engine: plans and counters are shared


def write_config(directory: Path, layers: int, tokens: int) -> Path:
    """A Qwen3.5-style config: the installed vLLM builds this model family from the combined
    (vision + text) config and runs it with ``language_model_only=True``, as the reference's
    harness does (``lcgemm/bench/prefill.py:60-68,104-106``); the vision tower is kept minimal."""
    pattern = ["linear_attention", "linear_attention", "linear_attention", "full_attention"]
    text = {
        "model_type": "qwen3_5_text",
        "hidden_size": 5120, "intermediate_size": 17408, "num_hidden_layers": layers,
        "num_attention_heads": 24, "num_key_value_heads": 4, "head_dim": 256,
        "linear_conv_kernel_dim": 4, "linear_key_head_dim": 128, "linear_value_head_dim": 128,
        "linear_num_key_heads": 16, "linear_num_value_heads": 48,
        "layer_types": [pattern[i % 4] for i in range(layers)], "full_attention_interval": 4,
        "vocab_size": 151936, "max_position_embeddings": max(8192, tokens) + 512, "rms_norm_eps": 1e-6,
        "hidden_act": "silu", "tie_word_embeddings": False, "attention_bias": False,
        "attention_dropout": 0.0, "partial_rotary_factor": 0.25,
        "rope_parameters": {"rope_type": "default", "rope_theta": 10000000.0, "partial_rotary_factor": 0.25,
                            "mrope_section": [11, 11, 10], "mrope_interleaved": True},
        "bos_token_id": 1, "eos_token_id": 2, "dtype": "bfloat16",
    }
    vision = {"model_type": "qwen3_5", "depth": 1, "hidden_size": 128, "intermediate_size": 256, "num_heads": 2,
              "out_hidden_size": 5120, "num_position_embeddings": 64, "patch_size": 16,
              "spatial_merge_size": 2, "temporal_patch_size": 2, "in_channels": 3}
    cfg = {"architectures": ["Qwen3_5ForConditionalGeneration"], "model_type": "qwen3_5",
           "text_config": text, "vision_config": vision, "tie_word_embeddings": False,
           "image_token_id": 151655, "video_token_id": 151656, "vision_start_token_id": 151652,
           "vision_end_token_id": 151653, "torch_dtype": "bfloat16"}
    directory.mkdir(parents=True, exist_ok=True)
    (directory / "config.json").write_text(json.dumps(cfg, indent=1))
    return directory


def run_arm(args) -> dict:
    import torch

    patch = None
    if args.arm == "optimized":
        from lcgemm.integrate import qwen_patch as patch

        patch.EXPECTED_LAYERS = args.layers
        patch.arm()
    from vllm import LLM, SamplingParams
    from vllm.inputs import TokensPrompt

    model_dir = write_config(Path(tempfile.mkdtemp(prefix="lcgemm_qwen35_dummy_")), args.layers, args.tokens)
    t0 = time.perf_counter()
    llm = LLM(model=str(model_dir), load_format="dummy", skip_tokenizer_init=True,
              max_model_len=args.tokens + 256, max_num_batched_tokens=args.tokens + 256, max_num_seqs=1,
              gpu_memory_utilization=args.gpu_memory_utilization, enable_prefix_caching=False,
              dtype="bfloat16", enforce_eager=args.enforce_eager, seed=0, language_model_only=True)
    build_s = time.perf_counter() - t0
    info = patch.install(llm, tokens=args.tokens) if patch else {}
    prompt = TokensPrompt(prompt_token_ids=[1000 + i % 5000 for i in range(args.tokens)])
    one = SamplingParams(max_tokens=1, temperature=0.0, detokenize=False)
    top = llm.generate([prompt], SamplingParams(max_tokens=1, temperature=0.0, logprobs=20, detokenize=False),
                       use_tqdm=False)[0].outputs[0]
    logprobs = sorted(((int(t), float(v.logprob)) for t, v in top.logprobs[0].items()), key=lambda kv: -kv[1])

    def call():
        llm.generate([prompt], one, use_tqdm=False)

    for _ in range(args.warmup):
        call()
    flush = torch.empty(256 << 20, dtype=torch.int8, device="cuda")
    before = patch.counts() if patch else {}
    wall = []
    for _ in range(args.runs):
        torch.cuda.synchronize()
        time.sleep(0.05)
        flush.zero_()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        call()
        torch.cuda.synchronize()
        wall.append((time.perf_counter() - t0) * 1e3)
    result = {"arm": args.arm, "tokens": args.tokens, "layers": args.layers,
              "layers_note": None if args.layers == 64 else f"shortened from 64 to {args.layers} layers",
              "weights": "dummy (vLLM load_format=dummy)", "enforce_eager": args.enforce_eager,
              "engine_build_s": build_s, "passes": len(wall), "wall_ms_median": statistics.median(wall),
              "wall_ms": wall, "generated": list(top.token_ids), "logprobs": logprobs,
              "patch": {k: v for k, v in info.items() if k != "describe"}}
    if patch:
        result.update(patch.check_calls(len(wall), since=before))
        result["counts"] = patch.counts()
    return result


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--arm", choices=("optimized", "stock"), default="optimized")
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--runs", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.40)
    ap.add_argument("--no-enforce-eager", dest="enforce_eager", action="store_false",
                    help="let vLLM compile and capture graphs (slow to start; the op is opaque to it either way)")
    args = ap.parse_args()
    try:
        print("RESULT_JSON " + json.dumps(run_arm(args)))
    except Exception as exc:            # the line a caller greps for, also on failure
        import traceback

        print("RESULT_JSON " + json.dumps({"arm": args.arm, "tokens": args.tokens, "layers": args.layers,
                                           "failed": "".join(traceback.format_exception_only(type(exc), exc))[-800:]}))
        raise


if __name__ == "__main__":
    main()
