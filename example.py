"""Minimal use of the public API (the reference's example.py:1-32 applies a chat template to two prompts and prints
the completions; a tokenizer is optional here, so token-id prompts work without any model files).

    python example.py                      # tiny random-init Qwen3 architecture, token-id prompts, CPU or GPU
    python example.py /path/to/Qwen3-0.6B  # a real Hugging Face checkpoint directory (string prompts)
"""
import sys

from tinyllmforge_b200 import LLM, SamplingParams, preset


def main():
    sp = SamplingParams(temperature=0.6, max_tokens=32)
    if len(sys.argv) > 1:
        llm = LLM(sys.argv[1], enforce_eager=True, tensor_parallel_size=1)
        prompts = ["introduce yourself", "list all prime numbers within 100"]
        if llm.tokenizer is not None and getattr(llm.tokenizer, "chat_template", None):
            prompts = [llm.tokenizer.apply_chat_template([{"role": "user", "content": p}], tokenize=False,
                                                         add_generation_prompt=True) for p in prompts]
    else:
        import torch
        on_gpu = torch.cuda.is_available()
        cfg = preset("qwen3-0.6b", num_hidden_layers=2, vocab_size=8192) if on_gpu else preset("tiny")
        llm = LLM("random-init", hf_config=cfg, load_format="dummy", skip_tokenizer_init=True, enforce_eager=True,
                  max_model_len=512, max_num_batched_tokens=1024, num_kvcache_blocks=64,
                  kvcache_block_size=256 if on_gpu else 16)
        prompts = [[11, 22, 33, 44, 55], [5, 4, 3, 2, 1, 0]]
    for prompt, out in zip(prompts, llm.generate(prompts, sp, use_tqdm=False)):
        print(f"prompt: {prompt!r}\ncompletion: {out['text']!r} {out['token_ids']}\n")
    llm.exit()


if __name__ == "__main__":
    main()
