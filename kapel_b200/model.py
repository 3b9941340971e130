"""The Python entry point, in the manner of Kapel's `kapel.Model` (crates/kapel-python/kapel.pyi:16-106).

    model = kapel_b200.Model("path/to/model", device="cuda", dtype="bf16")
    tokens = model.generate([2, 651, 6037], max_tokens=64)                  # greedy
    tokens = model.generate(prompt_ids, max_tokens=64, temperature=0.8, seed=7)
    for token in model.generate(prompt_ids, stream=True): ...

Option names and meanings are Kapel's. Prompts are token ids; a text prompt needs the folder's
tokenizer.json and the `tokenizers` package, which this engine does not itself provide. Quantized
weights and caches (`quantize`, `kv_cache` other than the compute dtype) are refused.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Iterator, List, Optional, Sequence, Union

from .engine.scheduler import EngineOptions, Event, Request, Scheduler
from .engine.step import Engine, parse_dtype
from .sampling import Sampling


class KapelError(RuntimeError):
    """A model that cannot be read, or a pass of a model that failed."""


_KV_NAMES = {"f32": "float32", "bf16": "bfloat16", "float32": "float32", "bfloat16": "bfloat16"}


class Model:
    def __init__(self, name, device: str = "cuda", dtype: Optional[str] = None, quantize: Optional[str] = None,
                 kv_cache: Optional[str] = None, revision: str = "main", max_tokens_cached: int = 65536,
                 max_sequences: int = 256, pages: Optional[int] = None, max_pass_tokens: int = 2048, strict: bool = False,
                 _engine: Optional[Engine] = None):
        """`pages` sizes every layer group's page pool (else `max_tokens_cached` / 16 pages);
        `max_pass_tokens` is the most tokens one pass of `generate` holds (the portions a prompt is
        cut into); `strict` makes a tensor of the file that the model does not name an error."""
        self.max_pass_tokens = int(max_pass_tokens)
        self.max_sequences = int(max_sequences)
        if quantize is not None:
            raise KapelError("quantized weights are not built in this engine")
        if not str(device).startswith("cuda"):
            raise KapelError(f"device {device!r}: this engine runs on a CUDA device only")
        self.dtype = parse_dtype(dtype or "bf16")
        if kv_cache is not None and parse_dtype(_KV_NAMES.get(kv_cache, kv_cache)) != self.dtype:
            raise KapelError(f"kv_cache {kv_cache!r}: the cache is kept in the compute dtype here")
        if _engine is not None:
            self.engine = _engine
            self.folder = None
        else:
            import torch

            index = int(str(device).split(":")[1]) if ":" in str(device) else torch.cuda.current_device() if torch.cuda.is_available() else 0
            if torch.cuda.is_available():
                torch.cuda.set_device(index)
            self.folder = Path(name)
            try:
                self.engine = Engine.from_dir(self.folder, dtype=self.dtype, max_tokens=max_tokens_cached, max_sequences=max_sequences,
                                              pages=pages, strict=strict)
            except (ValueError, OSError) as e:
                raise KapelError(str(e)) from e
        self._defaults = self._read_generation_config()
        self._tokenizer = None

    @classmethod
    def random(cls, config, seed: int = 0, dtype: str = "bf16", max_tokens_cached: int = 65536, max_sequences: int = 256,
               pages: Optional[int] = None, max_pass_tokens: int = 2048) -> "Model":
        """A model of `config` (config.json's dict, a typed configuration, the path of a config.json
        or the name of a preset) with random weights made on the device from `seed`."""
        if isinstance(config, (str, Path)):
            from .config import read_config_file

            config = read_config_file(config)
        engine = Engine.random(config, seed=seed, dtype=dtype, max_tokens=max_tokens_cached, max_sequences=max_sequences, pages=pages)
        return cls(None, dtype=dtype, max_sequences=max_sequences, max_pass_tokens=max_pass_tokens, _engine=engine)

    # ------------------------------------------------------------------ defaults
    def _read_generation_config(self):
        eos: List[int] = []
        sampling = Sampling()
        raw = self.engine.raw_config or {}
        gen = {}
        if self.folder is not None and (self.folder / "generation_config.json").is_file():
            try:
                gen = json.loads((self.folder / "generation_config.json").read_text())
            except json.JSONDecodeError:
                gen = {}
            sampling = Sampling.from_generation_config(gen)
        e = gen.get("eos_token_id", raw.get("eos_token_id"))
        if isinstance(e, int):
            eos = [e]
        elif isinstance(e, list):
            eos = [int(x) for x in e]
        return {"sampling": sampling, "eos": eos}

    # ------------------------------------------------------------------ text, if a tokenizer is there
    def _load_tokenizer(self):
        if self._tokenizer is None:
            if self.folder is None or not (self.folder / "tokenizer.json").is_file():
                raise KapelError("a text prompt needs tokenizer.json in the model folder; pass token ids instead")
            try:
                from tokenizers import Tokenizer
            except ImportError:
                raise KapelError("a text prompt needs the `tokenizers` package; pass token ids instead") from None
            self._tokenizer = Tokenizer.from_file(str(self.folder / "tokenizer.json"))
        return self._tokenizer

    def tokenize(self, text: str, add_special_tokens: bool = True) -> List[int]:
        return self._load_tokenizer().encode(text, add_special_tokens=add_special_tokens).ids

    def detokenize(self, ids: Sequence[int], skip_special_tokens: bool = False) -> str:
        return self._load_tokenizer().decode(list(ids), skip_special_tokens=skip_special_tokens)

    # ------------------------------------------------------------------ generation
    def _request(self, prompt, max_tokens, temperature, top_k, top_p, min_p, repetition_penalty, seed, stop,
                 ignore_eos=False) -> Request:
        d: Sampling = self._defaults["sampling"]
        sampling = Sampling(
            temperature=d.temperature if temperature is None else float(temperature),
            top_k=d.top_k if top_k is None else (int(top_k) or None),
            top_p=d.top_p if top_p is None else float(top_p),
            min_p=d.min_p if min_p is None else float(min_p),
            repetition_penalty=d.repetition_penalty if repetition_penalty is None else float(repetition_penalty),
            seed=0 if seed is None else int(seed),
        )
        stops = []
        for s in stop or ():
            stops.append(self.tokenize(s, add_special_tokens=False) if isinstance(s, str) else [int(t) for t in s])
        return Request(prompt=list(prompt), sampling=sampling, max_tokens=256 if max_tokens is None else int(max_tokens),
                       eos_ids=tuple(self._defaults["eos"]), ignore_eos=ignore_eos, stop=stops)

    def generate(self, prompt: Union[str, Sequence[int]], max_tokens: Optional[int] = None,
                 temperature: Optional[float] = None, top_k: Optional[int] = None, top_p: Optional[float] = None,
                 min_p: Optional[float] = None, repetition_penalty: Optional[float] = None, seed: Optional[int] = None,
                 stop: Optional[Sequence] = None, stream: bool = False, ignore_eos: bool = False):
        """The tokens generated after `prompt` (token ids in, token ids out; text in, text out).
        With `stream=True`, an iterator over them as they come."""
        as_text = isinstance(prompt, str)
        ids = self.tokenize(prompt) if as_text else [int(t) for t in prompt]
        request = self._request(ids, max_tokens, temperature, top_k, top_p, min_p, repetition_penalty, seed, stop, ignore_eos)
        it = self._run_one(request)
        if stream:
            return (self.detokenize([t]) for t in it) if as_text else it
        tokens = list(it)
        return self.detokenize(tokens, skip_special_tokens=True) if as_text else tokens

    def _run_one(self, request: Request) -> Iterator[int]:
        sched = Scheduler(self.engine, EngineOptions(max_pass_tokens=self.max_pass_tokens, max_sequences=1))
        self.last_scheduler = sched
        rid = sched.add(request)
        try:
            while sched.has_work():
                for ev in sched.step():
                    if ev.finish == "error":
                        raise KapelError(ev.error or "the pass failed")
                    if ev.token is not None and not (ev.finish == "eos"):
                        yield ev.token
        finally:
            sched.cancel(rid)

    def generate_batch(self, prompts: Sequence[Sequence[int]], max_tokens: Optional[int] = None,
                       temperature: Optional[float] = None, top_k: Optional[int] = None, top_p: Optional[float] = None,
                       min_p: Optional[float] = None, repetition_penalty: Optional[float] = None,
                       seed: Optional[int] = None, stop: Optional[Sequence] = None, ignore_eos: bool = False,
                       max_pass_tokens: int = 8192) -> List[List[int]]:
        """All prompts at once, as Kapel's `Batch` (crates/kapel-infer/src/batch.rs:20-88): 8192
        tokens a pass by default, and request i draws with seed + i."""
        sched = Scheduler(self.engine, EngineOptions(max_pass_tokens=max_pass_tokens, max_sequences=max(1, len(prompts))))
        ids = []
        for i, p in enumerate(prompts):
            s = (0 if seed is None else int(seed)) + i
            ids.append(sched.add(self._request(p, max_tokens, temperature, top_k, top_p, min_p, repetition_penalty, s, stop, ignore_eos)))
        out = {rid: [] for rid in ids}
        try:
            while sched.has_work():
                for ev in sched.step():
                    if ev.finish == "error":
                        raise KapelError(ev.error or "the pass failed")
                    if ev.token is not None and ev.finish != "eos":
                        out[ev.id].append(ev.token)
        finally:
            for rid in ids:
                sched.cancel(rid)
        self.last_stats = sched.stats()
        return [out[rid] for rid in ids]

    def scheduler(self, **options) -> Scheduler:
        """A scheduler of one's own over this model: `add`, `cancel`, `step`, `stats`."""
        options.setdefault("max_pass_tokens", self.max_pass_tokens)
        options.setdefault("max_sequences", self.max_sequences)
        return Scheduler(self.engine, EngineOptions(**options))

    def step(self, entries):
        """The step function itself: [(id, tokens, want)] -> float32 logits [wanted, vocab]."""
        return self.engine.step(entries)
