"""Child process of tests/test_vllm_plugin.py: runs upstream ``vllm.LLM`` with this package as the
platform plugin and prints what the test checks as one JSON line.

argv: <site dir with the installed distribution or ''> <model dir> <dtype> <mode>
mode: 'sync' | 'async' | 'preempt' | 'embeds' (a prompt-embedding request) | 'structured' (vLLM's structured outputs: a character-level
tokenizer is written next to the model and requests constrained to a choice run next to free ones)"""
import json
import os
import sys

site_dir, model_dir, dtype, mode = sys.argv[1:5]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
os.environ["VLLM_ENABLE_V1_MULTIPROCESSING"] = "0"
os.environ.setdefault("VLLM_LOGGING_LEVEL", "WARNING")
if site_dir:
    import site
    site.addsitedir(site_dir)            # processes the editable install's .pth file
else:
    sys.path.insert(0, ROOT)
    from vllm_ascend_b200.vllm_plugin import ensure_entry_points
    ensure_entry_points()

import numpy as np
import torch
from vllm import LLM, SamplingParams
from vllm.platforms import current_platform

if mode == "embeds":
    # a request that brings its input embeddings next to a request with token ids
    llm = LLM(model=model_dir, load_format="dummy", skip_tokenizer_init=True, dtype=dtype, max_model_len=256,
              max_num_seqs=8, max_num_batched_tokens=64, enable_prefix_caching=False, seed=0, enable_prompt_embeds=True)
    hidden = json.load(open(os.path.join(model_dir, "config.json")))["hidden_size"]
    pe = torch.randn(11, hidden, generator=torch.Generator().manual_seed(0)) * 0.05
    reqs = [{"prompt_embeds": pe}, {"prompt_token_ids": [5, 6, 7, 8, 9]}]
    outs = llm.generate(reqs, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True), use_tqdm=False)
    worker = llm.llm_engine.engine_core.engine_core.model_executor.driver_worker.worker
    from vllm_ascend_b200.config import ModelConfig
    from vllm_ascend_b200.engine.llm import LLM as OwnLLM
    from vllm_ascend_b200.engine.request import SamplingParams as OwnSP
    cfg = ModelConfig.from_hf_dict(json.load(open(os.path.join(model_dir, "config.json"))), dtype=dtype)
    cfg.name = os.path.basename(os.path.normpath(model_dir))
    own = OwnLLM(cfg, max_model_len=256, max_num_seqs=8, max_num_batched_tokens=64, seed=0,
                 block_size=worker.cfg.cache.block_size)
    want = [o.outputs[0].token_ids for o in own.generate(reqs, OwnSP(temperature=0.0, max_tokens=6, ignore_eos=True))]
    print("RESULT " + json.dumps({"platform": type(current_platform).__name__, "worker": type(worker).__name__,
                                  "got": [list(o.outputs[0].token_ids) for o in outs], "want": want}), flush=True)
    os._exit(0)

if mode == "structured":
    import string
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    from vllm.sampling_params import StructuredOutputsParams
    vocab = {"<pad>": 0, "<eos>": 1, "<unk>": 2}
    for ch in string.ascii_letters + string.digits + string.punctuation + " ":
        vocab.setdefault(ch, len(vocab))
    i = 0
    while len(vocab) < 1024:
        vocab[f"w{i}x"] = len(vocab)
        i += 1
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Split("", "isolated")
    tok.decoder = decoders.Fuse()
    PreTrainedTokenizerFast(tokenizer_object=tok, eos_token="<eos>", pad_token="<pad>",
                            unk_token="<unk>").save_pretrained(model_dir)
    cfg_path = os.path.join(model_dir, "config.json")
    hf = json.load(open(cfg_path))
    hf.update(eos_token_id=1, pad_token_id=0)
    json.dump(hf, open(cfg_path, "w"))
    llm = LLM(model=model_dir, tokenizer=model_dir, load_format="dummy", dtype=dtype, max_model_len=256, max_num_seqs=8,
              max_num_batched_tokens=64, enable_prefix_caching=False, seed=0)
    choices = ["yes", "no", "maybe"]
    constrained = SamplingParams(temperature=0.0, max_tokens=12,
                                 structured_outputs=StructuredOutputsParams(choice=choices))
    free = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(3, 1024, size=n).tolist() for n in (9, 20, 5, 33)]
    outs = llm.generate([{"prompt_token_ids": p} for p in prompts], [constrained, free, constrained, free], use_tqdm=False)
    worker = llm.llm_engine.engine_core.engine_core.model_executor.driver_worker.worker
    # the free requests alone: their tokens must not depend on sharing steps with constrained ones
    alone = llm.generate([{"prompt_token_ids": prompts[1]}, {"prompt_token_ids": prompts[3]}], free, use_tqdm=False)
    print("RESULT " + json.dumps({
        "platform": type(current_platform).__name__, "worker": type(worker).__name__,
        "texts": [o.outputs[0].text for o in outs], "choices": choices,
        "got": [list(o.outputs[0].token_ids) for o in outs],
        "free_alone": [list(o.outputs[0].token_ids) for o in alone]}), flush=True)
    os._exit(0)

kw = dict(model=model_dir, load_format="dummy", skip_tokenizer_init=True, dtype=dtype, max_model_len=256,
          max_num_seqs=8, max_num_batched_tokens=64, enable_prefix_caching=False, seed=0,
          async_scheduling=(mode == "async"))
on_gpu = torch.cuda.is_available()
if mode == "preempt":
    # too few blocks for every request to finish (pages: 128 tokens on a GPU, 16 on the host)
    kw["num_gpu_blocks_override"] = 6 if on_gpu else 20
llm = LLM(**kw)
rng = np.random.default_rng(0)
if mode != "preempt":
    lens, n_out = (20, 70, 33, 5), 8
elif on_gpu:
    lens, n_out = (100, 110, 90, 120), 60
else:
    lens, n_out = (40, 44, 36, 48), 40
prompts = [rng.integers(0, 1024, size=n).tolist() for n in lens]
outs = llm.generate([{"prompt_token_ids": p} for p in prompts],
                    SamplingParams(temperature=0.0, max_tokens=n_out, ignore_eos=True), use_tqdm=False)
got = [list(o.outputs[0].token_ids) for o in outs]

# the worker vLLM constructed
core = llm.llm_engine.engine_core.engine_core
worker = core.model_executor.driver_worker.worker
stats = dict(worker.stats)

# the same prompts through this package's own engine: same architecture, same seed, same weights
from vllm_ascend_b200 import _native
from vllm_ascend_b200.config import ModelConfig
from vllm_ascend_b200.engine.llm import LLM as OwnLLM
from vllm_ascend_b200.engine.request import SamplingParams as OwnSP
launches_under_vllm = int(_native.launch_counter[0]) + int(worker.runner.stats.get("graph_kernel_launches", 0))
cfg = ModelConfig.from_hf_dict(json.load(open(os.path.join(model_dir, "config.json"))), dtype=dtype)
cfg.name = os.path.basename(os.path.normpath(model_dir))
own = OwnLLM(cfg, max_model_len=256, max_num_seqs=8, max_num_batched_tokens=64, seed=0,
             block_size=worker.cfg.cache.block_size)
want = [o.outputs[0].token_ids for o in own.generate(prompts, OwnSP(temperature=0.0, max_tokens=n_out,
                                                                    ignore_eos=True))]
maps = open("/proc/self/maps").read()
print("RESULT " + json.dumps({
    "platform": type(current_platform).__name__, "worker": type(worker).__name__, "got": got, "want": want,
    "stats": stats, "native_mapped": "vllm_ascend_b200/_C.so" in maps, "launches": launches_under_vllm,
    "device": str(worker.device), "async": bool(worker._async),
    "installed": bool(site_dir)}), flush=True)
os._exit(0)
