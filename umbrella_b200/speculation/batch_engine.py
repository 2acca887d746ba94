"""BatchDecodingEngine: plain autoregressive decoding of static batches, for models that carry per-sequence state
(models/seq_model.py) instead of a rollback-able KV cache -- the engines next door verify token trees, which needs a
cache that can drop rejected rows; a recurrent state cannot, so these models decode one token per sequence per step
and get their throughput from batching.

Scheduling (the static batching of a serving loop): requests wait in a queue; a batch is formed from the head of the
queue, up to ``max_batch`` requests and ``max_tokens`` prompt tokens; its prompts are prefilled in ONE ragged step (no
padding), then every step decodes one token for each request still running; a request that hits EOS or its token
budget leaves the batch and gives its state slot back; when the batch is empty the next one is formed.  No request
joins a running batch.

``step(entries, end)`` is the primitive under both the generation loop and bin/trace_run: it maps request ids to
state slots (allocating one for an id it has not seen), runs ``model.forward`` and releases the slots of finished
requests.  Sampling is the framework's fused sampler (ops.sample: arg-max, or top-k / top-p at a temperature).

Engine-interface methods that only make sense with a draft model (``build_tree``) are no-ops here; ``verify`` is one
decoding step of the single interactive sequence.
"""
from __future__ import annotations

import time
from collections import deque

import torch

from .base import BaseEngine


class BatchDecodingEngine(BaseEngine):
    def __init__(self, target_model_name: str | None = None, draft_model_name: str | None = None, device: str = "cuda:0",
                 dtype="bfloat16", max_length: int | None = None, max_tokens: int = 0, max_batch: int = 8,
                 temperature: float = 0.0, topk: int = 32, topp: float = 0.9, seed: int = 0, tokenizer_name=None,
                 **config):
        self.target_model_name, self.device = target_model_name, device
        self.dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16,
                      "fp32": torch.float32}.get(dtype, dtype) if isinstance(dtype, str) else dtype
        self.max_length, self.max_tokens, self.max_batch = max_length, int(max_tokens), int(max_batch)
        self.temperature, self.topk, self.topp = float(temperature), int(topk), float(topp)
        self.seed = seed
        self.tokenizer_name = tokenizer_name
        self.config = config
        self.model = None
        self.tokenizer = None
        self.slot_of: dict = {}            # request id -> state slot
        self.queue: deque = deque()
        self._gen = None
        self._interactive = None           # (request id, tokens so far) of prefill / append / verify

    # ------------------------------------------------------------------ set-up
    def initialize(self, model=None, target_model=None, draft_model=None):
        model = model if model is not None else target_model
        if model is None:
            from ..models.auto_model import AutoModelLM
            model = AutoModelLM.from_pretrained(self.target_model_name, device=self.device, dtype=self.dtype,
                                                max_length=self.max_length, max_tokens=self.max_tokens,
                                                slots=self.max_batch)
            model.alloc(**{k: v for k, v in self.config.items() if k in ("synthetic", "synthetic_seed")})
        self.model = self.target_model = model
        self.eos_tokens = list(getattr(model, "eos_tokens", []))
        self._gen = torch.Generator(device=model.device).manual_seed(self.seed)
        if self.tokenizer_name:
            from transformers import AutoTokenizer
            self.tokenizer = AutoTokenizer.from_pretrained(self.tokenizer_name)
        return self

    def _set_eos(self, eos_tokens):
        self.eos_tokens = list(eos_tokens)

    def reset(self):
        for rid in list(self.slot_of):
            self.release(rid)
        self.queue.clear()
        self._interactive = None

    def validate_status(self):
        if self._interactive is None or self.max_length is None:
            return True
        return len(self._interactive[1]) < self.max_length

    def update_generation_args(self, **a):
        self.temperature = float(a.get("temperature", self.temperature))
        self.topp = float(a.get("topp", self.topp))
        self.topk = int(a.get("topk", self.topk))

    # ------------------------------------------------------------------ the step (scheduler primitive)
    def step(self, entries, end=()):
        """``entries``: [{"id", "tokens", "want"}] -- the next tokens of each request and the places among them whose
        logits are wanted; ``end``: ids finished after this step (their slots are given back).  -> fp32 [wanted, vocab]."""
        cache = self.model.cache
        batch = []
        for e in entries:
            rid = e["id"]
            if rid not in self.slot_of:
                self.slot_of[rid] = cache.alloc_slot()
            batch.append((self.slot_of[rid], e["tokens"], e.get("want", ())))
        logits = self.model.forward(batch)
        for rid in end:
            self.release(rid)
        return logits

    def release(self, rid):
        slot = self.slot_of.pop(rid, None)
        if slot is not None:
            self.model.cache.free_slot(slot)

    def sample(self, logits: torch.Tensor) -> torch.Tensor:
        """One token per row of fp32 logits: arg-max at temperature 0, else top-k / top-p sampling."""
        from .. import ops
        if self.temperature < 0.05:
            return ops.sample(logits, ops.UMB_SAMPLE_ARGMAX)
        u = torch.rand(logits.shape[0], generator=self._gen, device=logits.device, dtype=torch.float32)
        return ops.sample(logits, ops.UMB_SAMPLE_DYNAMIC, temperature=self.temperature, top_k=self.topk, top_p=self.topp,
                          uniforms=u)

    # ------------------------------------------------------------------ batches of requests
    def submit(self, rid, input_ids, max_new_tokens: int = 128):
        self.queue.append({"id": rid, "prompt": [int(t) for t in input_ids], "max_new": int(max_new_tokens), "out": []})

    def _form_batch(self):
        batch, tokens = [], 0
        while self.queue and len(batch) < self.max_batch:
            n = len(self.queue[0]["prompt"])
            if batch and self.max_tokens and tokens + n > self.max_tokens:
                break
            batch.append(self.queue.popleft())
            tokens += n
        return batch

    def run_queue(self) -> dict:
        """Serve every queued request; -> {request id: generated token ids}."""
        done = {}
        while self.queue:
            live = self._form_batch()
            logits = self.step([{"id": r["id"], "tokens": r["prompt"], "want": [len(r["prompt"]) - 1]} for r in live])
            while live:
                nxt = self.sample(logits).tolist()
                still, ended = [], []
                for r, t in zip(live, nxt):
                    r["out"].append(t)
                    over = t in self.eos_tokens or len(r["out"]) >= r["max_new"] or \
                        (self.max_length is not None and len(r["prompt"]) + len(r["out"]) >= self.max_length)
                    (ended if over else still).append(r)
                for r in ended:
                    done[r["id"]] = r["out"]
                    self.release(r["id"])
                live = still
                if live:
                    logits = self.step([{"id": r["id"], "tokens": [r["out"][-1]], "want": [0]} for r in live])
        return done

    def generate_batch(self, prompts, max_new_tokens: int = 128) -> list:
        """Greedy / sampled continuation of several prompts (lists of token ids) through the queue."""
        for i, p in enumerate(prompts):
            self.submit(("gen", i), p, max_new_tokens)
        out = self.run_queue()
        return [out[("gen", i)] for i in range(len(prompts))]

    # ------------------------------------------------------------------ single-sequence surface of the engine interface
    def _encode(self, text):
        if self.tokenizer is None:
            raise RuntimeError("no tokenizer: pass token ids (input_ids=...)")
        return self.tokenizer.encode(text)

    def _decode(self, ids):
        return self.tokenizer.decode(ids, skip_special_tokens=True) if self.tokenizer is not None else ""

    def prefill(self, text: str):
        return self._prefill(torch.tensor([self._encode(text)]))

    def append(self, text: str):
        ids = self._encode(text)
        return self._append(torch.tensor([ids[1:] if self.tokenizer.bos_token_id == ids[0] else ids]))

    def _prefill(self, input_ids):
        self.reset()
        self._interactive = ("interactive", [])
        return self._append(input_ids)

    def _append(self, input_ids):
        ids = torch.as_tensor(input_ids).reshape(-1).tolist()
        rid, toks = self._interactive
        if self.max_length is not None and len(toks) + len(ids) >= self.max_length:
            return False
        logits = self.step([{"id": rid, "tokens": ids, "want": [len(ids) - 1]}])
        toks += ids
        toks.append(int(self.sample(logits)[0]))          # the first committed token, fed by the next verify()
        return True

    def build_tree(self):
        return None

    def verify(self):
        rid, toks = self._interactive
        if toks[-1] in self.eos_tokens:
            return False
        logits = self.step([{"id": rid, "tokens": [toks[-1]], "want": [0]}])
        toks.append(int(self.sample(logits)[0]))
        return toks[-1] not in self.eos_tokens

    def speculative_decoding(self, max_new_tokens=128):
        start = len(self._interactive[1]) - 1
        torch.cuda.synchronize()
        t0, steps, go = time.time(), 0, True
        while go and len(self._interactive[1]) - start < max_new_tokens and self.validate_status():
            go = self.verify()
            steps += 1
        torch.cuda.synchronize()
        return self._interactive[1][start:], time.time() - t0, steps

    def generate(self, **api_args):
        self.update_generation_args(**api_args)
        ids, max_new = api_args.get("input_ids"), api_args.get("max_new_tokens", 128)
        if ids is None and api_args.get("context"):
            ids = self._encode(api_args["context"])
        if ids is None or len(ids) == 0 or max_new == 0:
            api_args.update(generated_text="", generated_tokens=[], avg_accept_tokens=0.0, time_per_output_token=0.0)
            return api_args
        torch.cuda.synchronize()
        t0 = time.time()
        out = self.generate_batch([list(ids)], max_new)[0]
        torch.cuda.synchronize()
        dt = time.time() - t0
        api_args.update(generated_text=self._decode(out), generated_tokens=out, avg_accept_tokens=1.0,
                        time_per_output_token=1000 * dt / max(len(out), 1), large_model_steps=len(out), decode_seconds=dt)
        return api_args

    def generate_stream(self, **api_args):
        out = self.generate(**api_args)
        yield out["generated_text"], f"{out['time_per_output_token']:.2f} ms/token"
