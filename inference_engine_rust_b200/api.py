"""The Python entry point, in the reference's manner: a loaded model that owns the weights
and the configuration (`LoadedModel::load`, src/loaded_model.rs:23-50) and a session that
owns the cache and runs prefill / decode / logits (`InferenceSession`,
src/engine/session.rs:12-74), plus the generation loop the reference keeps in its command
line (src/main.rs:97-116).
"""
from __future__ import annotations

import os
from typing import Iterable, List, Optional, Sequence, Union

import torch

from .config import ConfigError, config_from_dict, load_config, spec_of
from .engine import Engine, GenerationResult, Model, generate as _generate
from .parts.base import Runtime
from .sampling import Sampler, SamplingParams
from .weights import RandomSource, TensorSource, write_model_folder

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype in (torch.bfloat16, torch.float32):
            return dtype
    elif str(dtype) in _DTYPES:
        return _DTYPES[str(dtype)]
    raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}")


class LoadedModel:
    """Weights on the device plus the typed configuration they were built for."""

    def __init__(self, config, model: Model):
        self.config = config
        self.model = model
        self.spec = model.spec

    @classmethod
    def load(cls, model_dir: str, dtype="bfloat16", device="cuda:0",
             plain_kernels: bool = False, strict: bool = True) -> "LoadedModel":
        """A folder with config.json and model.safetensors (or sharded safetensors with their
        index).  `dtype`: bfloat16 = the kernels and precisions used for serving; float32 =
        the whole model in true 32-bit.  `strict=False` accepts a folder that carries tensors
        the model does not use (they are listed in `.model.ignored_tensors`); missing tensors
        and wrong shapes are errors either way.  A folder without `lm_head.weight` gets the
        embedding table as its output head."""
        config = load_config(model_dir)
        model = cls._build(config, dtype, device, plain_kernels)
        model.load(TensorSource(model_dir), where=model_dir, strict=strict)
        return cls(config, model)

    @classmethod
    def random(cls, config, seed: int = 0, dtype="bfloat16", device="cuda:0", std: float = 0.02,
               plain_kernels: bool = False, on_device: bool = False) -> "LoadedModel":
        """Seeded random weights for a typed configuration (or a config.json-style dict)."""
        if isinstance(config, dict):
            config = config_from_dict(config)
        model = cls._build(config, dtype, device, plain_kernels)
        model.load_random(seed, std, on_device=on_device)
        return cls(config, model)

    @staticmethod
    def _build(config, dtype, device, plain_kernels) -> Model:
        rt = Runtime(dtype=parse_dtype(dtype), device=torch.device(device), plain_only=plain_kernels)
        return Model(spec_of(config), rt)

    def session(self, **kw) -> "InferenceSession":
        return InferenceSession(self, **kw)


def write_random_model(model_dir: str, config, seed: int = 0, dtype="bfloat16",
                       std: float = 0.02) -> None:
    """The random-weights mode: writes config.json and model.safetensors for `config`
    (a typed configuration or a config.json-style dict) from a seed.  Runs on the host."""
    if isinstance(config, dict):
        config = config_from_dict(config)
    # which tensors exist follows from the parts; building them needs no device
    rt = Runtime(dtype=parse_dtype(dtype), device=torch.device("cpu"))
    expected = Model(spec_of(config), rt).expected_tensors()
    src = RandomSource(expected, seed, std, dtype=parse_dtype(dtype))
    write_model_folder(model_dir, config, {name: src.get(name) for name in expected})


class InferenceSession:
    """A cache for a loaded model and the steps that run against it.

    max_tokens     positions the cache holds over all live sequences (each rounded up to 64)
    max_sequences  slots; default: as many as there are pages, at most 1024
    use_graphs     replay captured CUDA graphs for one-token steps and short prompts (default)
    """

    def __init__(self, model: LoadedModel, max_tokens: int = 8192,
                 max_sequences: Optional[int] = None, max_seq_len: Optional[int] = None,
                 poison_cache: bool = False, use_graphs: bool = True):
        self.loaded = model
        self.engine = Engine(model.model, max_tokens=max_tokens, max_sequences=max_sequences,
                             max_seq_len=max_seq_len, poison_cache=poison_cache, use_graphs=use_graphs)
        self.max_tokens = max_tokens
        self._slots: List[int] = []

    # -- the reference's session calls, for a batch ------------------------------------------
    def reset(self) -> None:
        """Give back everything the session's current batch holds (src/engine/session.rs:40-42)."""
        for s in self._slots:
            self.engine.close_sequence(s)
        self._slots = []

    def prefill(self, prompts: Sequence[Sequence[int]], want="last") -> Optional[torch.Tensor]:
        """Start a batch: one prompt per sequence, unequal lengths allowed.  Returns the
        logits at the wanted places (default: each prompt's last token).  A prompt is run whole,
        from position 0: a sequence that already holds tokens can only go on one token at a
        time (`decode_tokens`), so a long prompt cannot be fed in portions and a running
        sequence cannot take a turn of several tokens at once (the engine refuses such a step
        with `StepError`; a windowed cache keeps only the newest positions of a prompt, which
        is right only if the prompt is attended to within the step that brings it)."""
        if self._slots:
            raise RuntimeError("a batch is running; reset() before starting another")
        if len(prompts) == 0:
            raise ValueError("prefill needs at least one prompt")
        try:
            for _ in prompts:                    # one by one: reset() gives back what was opened
                self._slots.append(self.engine.open_sequence())
            return self.engine.step(list(zip(self._slots, prompts)), want=want)
        except Exception:
            self.reset()
            raise

    def decode_tokens(self, tokens: Sequence[Optional[int]], want="last") -> Optional[torch.Tensor]:
        """One more token for each sequence of the batch; None ends that sequence (its slot is
        given back).  Logits come back in the order of the sequences that went on.  Exactly
        one token per sequence and call: several tokens for a running sequence are several
        calls."""
        if len(tokens) != len(self._slots):
            raise ValueError(f"{len(self._slots)} sequences are running, {len(tokens)} tokens given")
        entries, keep = [], []
        for slot, tok in zip(self._slots, tokens):
            if tok is None:
                self.engine.close_sequence(slot)
            else:
                entries.append((slot, [int(tok)]))
                keep.append(slot)
        self._slots = keep
        if not entries:
            return None
        return self.engine.step(entries, want=want)

    def decode_tokens_on_device(self, tokens: torch.Tensor, want="last") -> Optional[torch.Tensor]:
        """One more token for every sequence of the batch, the ids taken from device memory
        (int32 [sequences], e.g. what `Sampler.sample_device` returned): the step is launched
        without waiting for the ids on the host."""
        if not self._slots:
            raise RuntimeError("no batch is running; prefill() first")
        return self.engine.step_tokens_on_device(self._slots, tokens, want=want)

    def logits_last_token(self, logits: torch.Tensor) -> List[List[float]]:
        """Host copy of the logits a step returned (src/engine/session.rs:72-74)."""
        self.engine.check_device()
        return logits.float().cpu().tolist()

    # -- generation ---------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 20,
                 temperature: float = 0.0, seed: int = 0, stop_ids: Optional[Iterable[int]] = None,
                 max_batch: Optional[int] = None, request_ids: Optional[Sequence[int]] = None,
                 on_token=None, full: bool = False,
                 run_ahead: bool = True) -> Union[List[List[int]], List[GenerationResult]]:
        """Generated token ids for every prompt (host lists in, host lists out).  Stop ids
        default to the configuration's EOS; the stop token is not part of the output.
        `run_ahead` (default): chosen ids feed the next step from device memory and reach the
        host one step behind, so the device never waits for the host; results are the same."""
        if self._slots:
            raise RuntimeError("a batch started with prefill() is running; reset() first")
        spec = self.loaded.spec
        if stop_ids is None:
            stop_ids = [] if spec.eos_token_id is None else [spec.eos_token_id]
        sampler = Sampler(SamplingParams(temperature=temperature, seed=seed), self.engine.rt.err)
        cache = self.engine.cache
        res = _generate(self.engine, sampler, prompts, max_new_tokens, stop_ids=stop_ids,
                        max_tokens=cache.n_pages * cache.page_tokens, max_sequences=cache.n_slots,
                        max_seq_len=cache.max_seq_len, page_tokens=cache.page_tokens,
                        max_batch=max_batch, request_ids=request_ids, on_token=on_token,
                        run_ahead=run_ahead)
        self.engine.check_device()
        return res if full else [r.tokens for r in res]
