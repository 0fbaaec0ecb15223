"""The Python entry point under the reference's names.

``Qwen3InferenceConfig`` keeps the field names and meanings of
src/llm_pipeline/inference/qwen3_engine.py:21-83 where this engine has the thing they configure
(model path, device, dtype, generation and sampling defaults, ``max_batch_size``,
``block_size`` / ``num_blocks`` / ``max_sequence_length`` / ``memory_fraction`` of the paged
cache) and adds the token budget of the scheduler. Fields of the reference that switch between
its alternative code paths (``use_paged_attention``, ``enable_continuous_batching``,
``use_cuda_graphs``, ``use_torch_compile``, ``use_flash_attention``, tensor parallelism, prefix
and LRU caches) have no counterpart: there is one path, paged and continuously batched.

``Qwen3InferenceEngine.generate(prompt, max_tokens, temperature, top_k, top_p)`` follows
:311-350: a string gives a string, a list of strings gives a list. Prompts may also be lists of
token ids (a model folder with random weights has no tokenizer); the result is then a list of
token ids per prompt.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional, Sequence, Union

import torch

from .engine.generate import GenerationEngine, GenerationResult
from .sampling import SamplingConfig

_DTYPES = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp32": torch.float32, "float32": torch.float32}


@dataclass
class Qwen3InferenceConfig:
    model_path: str
    device: str = "cuda:0"
    dtype: Union[torch.dtype, str] = torch.bfloat16
    # generation (reference :36-49)
    max_length: int = 2048
    max_new_tokens: int = 512
    temperature: float = 1.0
    top_p: float = 0.9
    top_k: int = 50
    repetition_penalty: float = 1.0
    typical_p: float = 1.0
    min_p: float = 0.0
    do_sample: bool = True
    pad_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    seed: int = 0
    # batching and cache (reference :52-71)
    max_batch_size: int = 8
    block_size: int = 16
    num_blocks: Optional[int] = None
    max_sequence_length: int = 2048
    memory_fraction: float = 0.8
    # scheduler
    max_num_batched_tokens: int = 2048
    max_prefill_chunk: Optional[int] = None


def resolve_dtype(dtype: Union[torch.dtype, str]) -> torch.dtype:
    if isinstance(dtype, str):
        if dtype not in _DTYPES:
            raise ValueError(f"dtype {dtype!r} is not supported; this engine computes in bf16 or fp32")
        return _DTYPES[dtype]
    if dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"dtype {dtype} is not supported; this engine computes in bfloat16 or float32")
    return dtype


class Qwen3InferenceEngine:
    def __init__(self, config: Qwen3InferenceConfig):
        self.config = config
        self.device = torch.device(config.device)
        dtype = resolve_dtype(config.dtype)
        sampling = SamplingConfig(temperature=config.temperature, top_k=config.top_k, top_p=config.top_p,
                                  repetition_penalty=config.repetition_penalty, typical_p=config.typical_p,
                                  min_p=config.min_p, do_sample=config.do_sample, pad_token_id=config.pad_token_id,
                                  eos_token_id=config.eos_token_id, seed=config.seed)
        self.engine = GenerationEngine.from_folder(
            config.model_path, device=config.device, dtype=dtype, page_size=config.block_size,
            num_pages=config.num_blocks, memory_fraction=config.memory_fraction, max_num_seqs=config.max_batch_size,
            max_num_batched_tokens=config.max_num_batched_tokens, max_model_len=config.max_sequence_length,
            max_prefill_chunk=config.max_prefill_chunk, sampling=sampling)
        self.model_config = self.engine.config
        self._continuous: dict = {}              # add_continuous_request: id -> (prompt as given, time it was added)
        self._continuous_done: dict = {}         # id -> time its result was first seen finished
        self.tokenizer = self._load_tokenizer(config.model_path)
        if self.tokenizer is not None:
            if config.pad_token_id is None:
                config.pad_token_id = getattr(self.tokenizer, "pad_token_id", None)
            if config.eos_token_id is None:
                config.eos_token_id = getattr(self.tokenizer, "eos_token_id", None)

    @staticmethod
    def _load_tokenizer(path: str):
        """The tokenizer of the model folder, if it has one (the reference loads it with
        ``AutoTokenizer``, src/llm_pipeline/models/qwen3/factory.py:97)."""
        if not any(os.path.isfile(os.path.join(path, f)) for f in ("tokenizer.json", "tokenizer_config.json", "vocab.json")):
            return None
        from transformers import AutoTokenizer

        return AutoTokenizer.from_pretrained(path, local_files_only=True)

    def _eos_ids(self) -> List[int]:
        ids = set(self.model_config.eos_token_ids())
        if self.config.eos_token_id is not None:
            ids.add(int(self.config.eos_token_id))
        return sorted(ids)

    def generate(self, prompt, max_tokens: Optional[int] = None, temperature: Optional[float] = None,
                 top_k: Optional[int] = None, top_p: Optional[float] = None, **kwargs):
        single = isinstance(prompt, str) or (isinstance(prompt, Sequence) and len(prompt) > 0
                                             and isinstance(prompt[0], int))
        prompts = [prompt] if single else list(prompt)
        as_text = all(isinstance(p, str) for p in prompts)
        if as_text:
            if self.tokenizer is None:
                raise ValueError("the model folder has no tokenizer; pass prompts as lists of token ids")
            token_prompts = [self.tokenizer(p)["input_ids"] for p in prompts]
        else:
            token_prompts = [list(p) for p in prompts]
        results = self.generate_ids(token_prompts, max_tokens, temperature, top_k, top_p, **kwargs)
        if as_text:
            outs = [self.tokenizer.decode(r.token_ids, skip_special_tokens=True) for r in results]
        else:
            outs = [r.token_ids for r in results]
        return outs[0] if single else outs

    def generate_ids(self, prompts: Sequence[Sequence[int]], max_tokens: Optional[int] = None,
                     temperature: Optional[float] = None, top_k: Optional[int] = None, top_p: Optional[float] = None,
                     **kwargs) -> List[GenerationResult]:
        max_tokens = max_tokens or self.config.max_new_tokens
        results: List[GenerationResult] = []
        prompts = list(prompts)
        eos = self._eos_ids()
        base = self.engine.sampler.config.merged({"temperature": temperature, "top_k": top_k, "top_p": top_p, **kwargs})
        from dataclasses import replace
        ids = [self.engine.add_request(p, max_tokens, replace(base, seed=base.seed + i), eos_token_ids=eos,
                                       ignore_eos=bool(kwargs.get("ignore_eos", False)))
               for i, p in enumerate(prompts)]
        mine = [self.engine._requests[i] for i in ids]
        # until every request of THIS call is finished: requests of other callers (an open stream, add_request) may
        # finish meanwhile and are none of this call's business
        while any(r.status != "finished" for r in mine):
            self.engine.step()
        for i, r in zip(ids, mine):
            self.engine._requests.pop(i, None)
            results.append(GenerationResult(i, r.prompt, r.output, r.finish_reason, r.preemptions))
        return results

    def batch_generate(self, prompts, **kwargs):
        """The reference's batch call (qwen3_engine.py:552-554): a list in, a list out. Here the prompts
        share steps (continuous batching) instead of one padded rectangle."""
        return self.generate(list(prompts), **kwargs)

    def continuous_batch_generate(self, prompts, **kwargs):
        """The reference's continuous-batching call (qwen3_engine.py:562-575). This engine always batches
        continuously, so it is the same as ``generate`` on a list."""
        return self.generate(list(prompts), **kwargs)

    def stream_generate(self, prompt, max_tokens: Optional[int] = None, temperature: Optional[float] = None,
                        top_k: Optional[int] = None, top_p: Optional[float] = None, **kwargs):
        """Yield the generation piece by piece as it is produced (qwen3_engine.py:556-560): decoded text
        pieces for a string prompt, token ids for a prompt of token ids."""
        as_text = isinstance(prompt, str)
        if as_text and self.tokenizer is None:
            raise ValueError("the model folder has no tokenizer; pass the prompt as a list of token ids")
        ids = self.tokenizer(prompt)["input_ids"] if as_text else list(prompt)
        base = self.engine.sampler.config.merged({"temperature": temperature, "top_k": top_k, "top_p": top_p, **kwargs})
        req_id = self.engine.add_request(ids, max_tokens or self.config.max_new_tokens, base, eos_token_ids=self._eos_ids(),
                                         ignore_eos=bool(kwargs.get("ignore_eos", False)))
        request = self.engine._requests[req_id]
        sent = 0
        text_so_far = ""
        try:
            while True:
                # what the request has produced since the last look: in this call's own steps, or in the steps of
                # another caller of the engine while this generator was not being read
                # (the count is taken before every yield: the caller may run the engine before it comes back)
                if as_text and len(request.output) > sent:
                    sent = len(request.output)
                    text = self.tokenizer.decode(request.output[:sent], skip_special_tokens=True)
                    piece, text_so_far = text[len(text_so_far):], text
                    if piece:
                        yield piece
                    continue
                if not as_text and len(request.output) > sent:
                    sent += 1
                    yield request.output[sent - 1]
                    continue
                if request.status == "finished":
                    break
                self.engine.step()
        finally:
            # a caller that stops iterating (or closes the generator) must not leave the request running with its pages
            if request.status != "finished":
                self.engine.abort(req_id)
            self.engine._requests.pop(req_id, None)

    def get_stats(self):
        return self.engine.stats()

    # -- the reference's calls around its batcher and its caches (qwen3_engine.py:614-712) -------------------------
    # Here there is one engine, always paged and continuously batched, and no thread of its own: a request that was
    # added runs in the steps of whoever drives the engine next (a generate call, a stream, ``get_continuous_result``).
    def start_continuous_batching(self) -> None:
        """Nothing to start (qwen3_engine.py:623-626 starts the batcher's thread)."""

    def stop_continuous_batching(self) -> None:
        """Nothing to stop (qwen3_engine.py:628-631)."""

    def add_continuous_request(self, prompt, max_tokens: int = 50, **kwargs) -> str:
        """Queue a request and return at once (qwen3_engine.py:633-649). ``prompt``: a string (with a tokenizer in the
        model folder) or a list of token ids. The id is of the reference's form."""
        import time
        as_text = isinstance(prompt, str)
        if as_text and self.tokenizer is None:
            raise ValueError("the model folder has no tokenizer; pass the prompt as a list of token ids")
        ids = self.tokenizer(prompt)["input_ids"] if as_text else list(prompt)
        ignore_eos = bool(kwargs.pop("ignore_eos", False))
        base = self.engine.sampler.config.merged(kwargs)
        request_id = f"req_{id(prompt)}_{int(time.time() * 1000)}_{len(self._continuous)}"
        self.engine.add_request(ids, max_tokens, base, eos_token_ids=self._eos_ids(), ignore_eos=ignore_eos, req_id=request_id)
        self._continuous[request_id] = (prompt, time.time())
        return request_id

    def get_continuous_result(self, request_id: str):
        """The finished request as the reference's dictionary (continuous_batching.py:286-293), or None while it is
        not finished; a call that finds it unfinished runs one step of the engine first."""
        import time
        if request_id not in self._continuous:
            raise KeyError(f"no continuous request {request_id!r}")
        request = self.engine._requests[request_id]
        if request.status != "finished":
            self.engine.step()
            if request.status != "finished":
                return None
        prompt, started = self._continuous[request_id]
        finished = self._continuous_done.setdefault(request_id, time.time())
        text = self.tokenizer.decode(request.output, skip_special_tokens=True) if self.tokenizer is not None else ""
        return {"request_id": request_id, "prompt": prompt, "generated_text": text, "generated_tokens": list(request.output),
                "latency_ms": (finished - started) * 1000, "tokens_generated": len(request.output),
                "finish_reason": request.finish_reason}

    def get_continuous_stats(self):
        """Counters of scheduler and cache (the reference's batcher counts the same things, continuous_batching.py:448-463)."""
        return self.engine.stats()

    def get_kv_cache_stats(self):
        """Pages free, used, at most used and used again per group; live requests (qwen3_engine.py:614-616)."""
        return self.engine.cache.stats()

    def clear_kv_cache(self) -> None:
        """Give every page back: whatever is queued or running is aborted (qwen3_engine.py:618-621)."""
        self.cleanup()

    def get_optimization_stats(self):
        """The reference's switches (qwen3_engine.py:672-695) as they are here: always on, or not built."""
        runner = self.engine.runner
        return {"torch_compile_enabled": False, "cuda_graphs_enabled": bool(runner.use_graphs),
                "paged_attention_enabled": True, "flash_attention_enabled": False, "prefix_caching_enabled": False,
                "tensor_parallel_enabled": False, "one_step_ahead": bool(self.engine.lookahead),
                "cuda_graphs": {"num_graphs": len(runner._graphs), "replays": runner.graph_replays},
                "paged_attention": self.engine.cache.stats()}

    def get_model_info(self):
        """Sizes and parameter counts from the model's configuration (models/qwen3/factory.py:132-166)."""
        c = self.model_config
        info = {"model_type": getattr(c, "model_type", "qwen3"), "vocab_size": c.vocab_size, "hidden_size": c.hidden_size,
                "num_layers": c.num_hidden_layers, "num_attention_heads": c.num_attention_heads,
                "num_key_value_heads": c.num_key_value_heads, "intermediate_size": c.intermediate_size,
                "max_position_embeddings": c.max_position_embeddings, "head_dim": c.head_dim,
                "torch_dtype": str(self.engine.dtype), "use_cache": True, "tie_word_embeddings": bool(c.tie_word_embeddings)}
        info.update(c.parameter_counts())
        return info

    def estimate_memory_usage(self):
        """Bytes of the weights in the engine's type and the reference's rule of thumb for the GPU
        (models/qwen3/factory.py:168-211), with what a token of context costs in this engine's cache."""
        info = self.get_model_info()
        bytes_per_param = 4 if self.engine.dtype == torch.float32 else 2
        memory_mb = info["total_parameters"] * bytes_per_param / (1024 * 1024)
        memory_gb = memory_mb / 1024
        from .cache import CacheManager
        per_page = sum(CacheManager.bytes_per_page(self.engine.model.cache_specs(), self.engine.cache.page_size, self.engine.dtype))
        return {**{k: v for k, v in info.items() if k.endswith("parameters") or k.endswith("_per_layer")},
                "memory_mb": memory_mb, "memory_gb": memory_gb, "model_memory_mb": memory_mb, "model_memory_gb": memory_gb,
                "bytes_per_param": bytes_per_param, "dtype": str(self.engine.dtype),
                "recommended_gpu_memory_gb": max(memory_gb * 1.5, memory_gb + 1.0),
                "kv_cache_bytes_per_token": per_page // self.engine.cache.page_size}

    def cleanup(self) -> None:
        """Abort whatever is still queued or running and give its pages back."""
        for request in list(self.engine.scheduler.running) + list(self.engine.scheduler.waiting):
            self.engine.abort(request.req_id)
        for req_id in list(self.engine._requests):
            self.engine.abort(req_id)                        # requests whose last token is still on its way
        self.engine.drain()
        self.engine._requests.clear()
        self._continuous.clear()
        self._continuous_done.clear()
