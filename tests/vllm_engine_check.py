"""Helper of tests/test_vllm_engine_gpu.py (run as a child process so that the engine's process group, memory pool
and environment stay out of the test process): starts a vLLM engine in this process on a small random-weight Llama
of the SmolLM2 shape family, generates greedily with the stock forward and again with the decode router installed,
and prints one JSON line with the comparison."""
import json
import os
import sys
import tempfile
from pathlib import Path

os.environ["VLLM_ENABLE_V1_MULTIPROCESSING"] = "0"          # engine core in this process: the patch must reach the model
os.environ.setdefault("VLLM_LOGGING_LEVEL", "ERROR")
sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

CONFIG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 576, "intermediate_size": 1536,
    "num_hidden_layers": 4, "num_attention_heads": 9, "num_key_value_heads": 3, "head_dim": 64, "vocab_size": 49152,
    "max_position_embeddings": 2048, "rms_norm_eps": 1e-05, "rope_theta": 100000.0, "hidden_act": "silu",
    "tie_word_embeddings": True, "torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 2,
    "attention_bias": False, "mlp_bias": False,
}


def main():
    import torch

    try:
        from vllm import LLM, SamplingParams
        from vllm.model_executor.models.llama import LlamaModel
    except Exception as e:                       # vLLM missing or not importable on this box
        print(json.dumps({"skip": f"vllm not importable: {type(e).__name__}: {e}"[:300]}))
        return
    with tempfile.TemporaryDirectory() as d:
        (Path(d) / "config.json").write_text(json.dumps(CONFIG))
        try:
            llm = LLM(model=d, load_format="dummy", dtype="bfloat16", enforce_eager=True, skip_tokenizer_init=True,
                      max_model_len=512, gpu_memory_utilization=0.2, seed=0, max_num_seqs=8, attention_backend="FLASH_ATTN")
        except Exception as e:
            print(json.dumps({"skip": f"engine did not start: {type(e).__name__}: {e}"[:300]}))
            return

        def init(model):                          # seeded weights instead of the dummy loader's near-zero ones
            g = torch.Generator(device="cuda").manual_seed(1)
            with torch.no_grad():
                for name, p in model.named_parameters():
                    r = torch.randn(p.shape, generator=g, device="cuda", dtype=torch.float32)
                    p.copy_(1.0 + 0.1 * r if "norm" in name else 0.02 * r)
            cache = model.model.layers[0].self_attn.attn.kv_cache
            return list(cache.shape)

        try:
            run_cases(llm, init, SamplingParams, LlamaModel)
        except Exception as e:                   # a failure past this point is the router's, not the engine's
            import traceback

            print(json.dumps({"error": f"{type(e).__name__}: {e}"[:300], "trace": traceback.format_exc()[-1500:]}))


def run_cases(llm, init, SamplingParams, LlamaModel):
    cache_shape = llm.apply_model(init)[0]
    sp = SamplingParams(temperature=0.0, max_tokens=8, logprobs=5, detokenize=False)
    from prime_kernels_b200 import decode_backend as db

    cases = []
    for n in (3, 6):                          # CUDA-core kernel (3 requests), tensor-core kernel (6)
        prompts = [{"prompt_token_ids": [(7 * i + 3 * j + 11) % 49152 for j in range(5 + 3 * i)]} for i in range(n)]
        stock = llm.generate(prompts, sp, use_tqdm=False)
        original = db.install_into_vllm()
        db.stats.clear()
        routed = llm.generate(prompts, sp, use_tqdm=False)
        stats = dict(db.stats)
        if original is not None:
            LlamaModel.forward = original
        worst, equal_tokens, total_tokens = 0.0, 0, 0
        for a, b in zip(stock, routed):
            ta, tb = a.outputs[0].token_ids, b.outputs[0].token_ids
            total_tokens += len(ta)
            for step, (x, y) in enumerate(zip(a.outputs[0].logprobs, b.outputs[0].logprobs)):
                if ta[step] != tb[step]:
                    break
                equal_tokens += 1
                worst = max(worst, abs(x[ta[step]].logprob - y[tb[step]].logprob))
        cases.append({"requests": n, "stats": stats, "equal_tokens": equal_tokens, "total_tokens": total_tokens,
                      "max_logprob_diff": worst})
    print(json.dumps({"cache_shape": cache_shape, "cases": cases}))


if __name__ == "__main__":
    main()
