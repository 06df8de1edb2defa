"""Model factories with the reference's signatures (``moshi/moshi/models/loaders.py:145-446``).

``get_mimi`` / ``get_moshi_lm`` / ``CheckpointInfo`` accept what the reference accepts on this path
(safetensors checkpoints with the reference's key names, the JSON LM config, the nested Mimi config
dict) and return B200-backed ``MimiModel`` / ``LMModel`` objects.  With ``filename=None`` the
reference returns an un-initialised model; here that means seeded synthetic weights
(``moshi_b200.synth``), which is also what the tests and the bench use offline.
"""
from __future__ import annotations

import json
import typing as tp
from dataclasses import dataclass, field
from pathlib import Path

import torch

from ..config import DECODER_ARCHITECTURES, DecoderLMConfig, LMConfig, MimiConfig
from ..synth import iter_synth_lm_tensors, synth_mimi_state_dict
from .compression import MimiModel
from .decoder_lm import DecoderLM
from .lm import LMModel

SAMPLE_RATE = 24000
FRAME_RATE = 12.5
TEXT_TOKENIZER_NAME = "tokenizer_spm_32k_3.model"
MOSHI_NAME = "model.safetensors"
MOSHI_Q8_NAME = "model.q8.safetensors"
MIMI_NAME = "tokenizer-e351c8d8-checkpoint125.safetensors"
DEFAULT_REPO = "kyutai/moshiko-pytorch-bf16"


def _is_safetensors(path: Path | str) -> bool:
    return Path(path).suffix in (".safetensors", ".sft", ".sfts")


def get_mimi(filename: str | Path | None, mimi_config: dict | None = None,
             device: torch.device | str = "cuda", num_codebooks: int = 8,
             synth_seed: int = 1234) -> MimiModel:
    """``loaders.get_mimi`` (loaders.py:323-363)."""
    cfg = MimiConfig.from_reference_dict(mimi_config, num_codebooks=num_codebooks)
    if filename is None:
        sd = synth_mimi_state_dict(cfg, seed=synth_seed)
    elif _is_safetensors(filename):
        from safetensors.torch import load_file
        sd = load_file(str(filename), device="cpu")
    else:
        sd = torch.load(filename, "cpu")["model"]
    model = MimiModel(cfg, sd, device=device)
    model.set_num_codebooks(num_codebooks)
    return model


def get_moshi_lm(filename: str | Path | None, lm_kwargs: dict | None = None,
                 device: torch.device | str = "cuda", dtype: torch.dtype = torch.bfloat16,
                 lora_weights: str | Path | None = None, fuse_lora: bool = False,
                 lm_kwargs_overrides: dict = {}, synth_seed: int = 4242,
                 synth_device: str | torch.device | None = None) -> LMModel:
    """``loaders.get_moshi_lm`` (loaders.py:366-446).  Checkpoints: ``model.safetensors`` (bf16), ``model.q8.safetensors``
    (loaders.py:33: every nn.Linear stored as a QLinear, ``weight`` int8 + ``weight_scb`` float32; needs ``quantize=True`` in the
    kwargs, like the reference), ``.gguf`` (the Rust stack's quantised form, F32 / F16 / BF16 / Q8_0 tensors under candle's names:
    ``moshi_b200/models/gguf.py``) and legacy ``.pt`` packages; packed ``in_proj_weight`` names are split (transformer.py:422-446).
    LoRA adapters are fused offline (loaders.py:512-513)."""
    if lora_weights is not None:
        raise ValueError("LoRA checkpoints are fused offline (loaders.py:512-513); pass fused weights")
    kwargs = dict(LMConfig().to_reference_kwargs() if lm_kwargs is None else lm_kwargs)
    kwargs.update(lm_kwargs_overrides)
    for k in ("lora", "lora_rank", "lora_scaling"):
        kwargs.pop(k, None)
    cfg = LMConfig.from_dict(kwargs)
    if filename is None:
        tensors: tp.Any = iter_synth_lm_tensors(cfg, seed=synth_seed, device=synth_device or "cpu", dtype=dtype)
    elif _is_safetensors(filename):
        from safetensors import safe_open

        def _stream():
            with safe_open(str(filename), framework="pt", device="cpu") as f:
                for key in f.keys():
                    yield key, f.get_tensor(key)
        tensors = _stream()
    elif Path(filename).suffix == ".gguf":
        # the Rust stack's quantised checkpoints (rust/moshi-core/src/nn.rs:9-116): candle tensor names, Q8_0 blocks dequantised
        from .gguf import read_gguf
        _, tensors = read_gguf(filename)
    else:
        tensors = torch.load(filename, "cpu")["fsdp_best_state"]["model"]
    return LMModel(cfg, tensors, device=device, dtype=dtype)


def read_safetensors(path: str | Path) -> tp.Iterator[tuple[str, torch.Tensor]]:
    """Streams (name, tensor) out of a safetensors file: 8-byte little-endian header length, a JSON header (name -> dtype, shape,
    data_offsets), then the data.  bf16 / f16 / f32 / i32 / i64 / u8 / i8 tensors."""
    import numpy as np
    kinds = {"BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F32": (torch.float32, 4), "I32": (torch.int32, 4),
             "I64": (torch.int64, 8), "U8": (torch.uint8, 1), "I8": (torch.int8, 1)}
    with open(path, "rb") as f:
        n = int.from_bytes(f.read(8), "little")
        header = json.loads(f.read(n))
        base = 8 + n
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            if meta["dtype"] not in kinds:
                raise ValueError(f"{path}: tensor {name!r} has dtype {meta['dtype']}")
            dt, _ = kinds[meta["dtype"]]
            lo, hi = meta["data_offsets"]
            f.seek(base + lo)
            raw = np.frombuffer(f.read(hi - lo), dtype=np.uint8).copy()
            yield name, torch.from_numpy(raw).view(dt).reshape(meta["shape"])


def model_class(config: dict):
    """The model registry: which class serves a ``config.json``.  Text-only decoder LMs name their ``architecture``; the Moshi LM's
    JSON (``configs/moshi_7b_202409.json``) has none and is recognised by its own keys."""
    arch = config.get("architecture")
    if arch in DECODER_ARCHITECTURES:
        return DecoderLM
    if arch is None and "dep_q" in config and "n_q" in config:
        return LMModel
    raise ValueError(f"no model class for architecture {arch!r} (decoder LMs: {sorted(DECODER_ARCHITECTURES)})")


def get_decoder_lm(model_dir: str | Path | None, config: dict | DecoderLMConfig | None = None, device: torch.device | str = "cuda",
                   dtype: torch.dtype = torch.bfloat16, synth_seed: int = 99, use_tc: bool = True) -> DecoderLM:
    """A text-only decoder LM from a folder holding ``config.json`` + ``model.safetensors``; with ``model_dir=None`` the given
    configuration gets seeded synthetic weights (``moshi_b200.synth.iter_synth_decoder_tensors``), as ``get_moshi_lm`` does."""
    if model_dir is not None:
        raw = json.loads((Path(model_dir) / "config.json").read_text())
        if model_class(raw) is not DecoderLM:
            raise ValueError(f"{model_dir}: not a decoder LM configuration")
        cfg = DECODER_ARCHITECTURES[raw["architecture"]].from_dict(raw)
        tensors: tp.Any = read_safetensors(Path(model_dir) / "model.safetensors")
    else:
        if config is None:
            raise ValueError("get_decoder_lm: give a model folder or a configuration")
        cfg = config if isinstance(config, DecoderLMConfig) else DecoderLMConfig.from_dict(config)
        from ..synth import iter_synth_decoder_tensors
        tensors = iter_synth_decoder_tensors(cfg, seed=synth_seed, device=device)
    return DecoderLM(cfg, tensors, device=device, dtype=dtype, use_tc=use_tc)


def get_model(model_dir: str | Path, device: torch.device | str = "cuda", dtype: torch.dtype = torch.bfloat16, **kwargs):
    """Model folder -> the registered class for its ``config.json``."""
    raw = json.loads((Path(model_dir) / "config.json").read_text())
    cls = model_class(raw)
    if cls is DecoderLM:
        return get_decoder_lm(model_dir, device=device, dtype=dtype, **kwargs)
    weights = Path(model_dir) / MOSHI_NAME
    return get_moshi_lm(weights if weights.exists() else None, lm_kwargs=raw, device=device, dtype=dtype, **kwargs)


@dataclass
class CheckpointInfo:
    """``loaders.CheckpointInfo`` (loaders.py:145-316) for local files; hub download needs a network."""
    moshi_weights: Path | None
    mimi_weights: Path | None
    tokenizer: Path | None
    lm_config: dict | None = None
    raw_config: dict | None = None
    mimi_config: dict | None = None
    model_type: str = "moshi"
    lora_weights: Path | None = None
    lm_gen_config: dict = field(default_factory=dict)
    tts_config: dict = field(default_factory=dict)
    stt_config: dict = field(default_factory=dict)
    model_id: dict = field(default_factory=dict)

    @staticmethod
    def from_hf_repo(hf_repo: str, moshi_weights=None, mimi_weights=None, tokenizer=None, config_path=None,
                     mimi_config_path=None, lora_weights=None, revision=None) -> "CheckpointInfo":
        from huggingface_hub import hf_hub_download

        def fetch(name_or_path, default_name):
            if name_or_path is not None:
                return Path(name_or_path)
            return Path(hf_hub_download(hf_repo, default_name, revision=revision))
        lm_config = raw = None
        names = {"moshi": MOSHI_NAME, "mimi": MIMI_NAME, "tok": TEXT_TOKENIZER_NAME}
        if config_path is None:
            try:
                config_path = hf_hub_download(hf_repo, "config.json", revision=revision)
            except Exception:
                config_path = None
        gen_cfg: dict = {}
        if config_path is not None:
            raw = json.loads(Path(config_path).read_text())
            lm_config = dict(raw)
            names["moshi"] = lm_config.pop("moshi_name", MOSHI_NAME)
            names["mimi"] = lm_config.pop("mimi_name", MIMI_NAME)
            names["tok"] = lm_config.pop("tokenizer_name", TEXT_TOKENIZER_NAME)
            for k in ("mimi_config_name", "lora_name", "tts_config", "stt_config", "model_id"):
                lm_config.pop(k, None)
            lm_config.pop("model_type", None)
            gen_cfg = lm_config.pop("lm_gen_config", {})
        mimi_cfg = json.loads(Path(mimi_config_path).read_text()) if mimi_config_path else None
        return CheckpointInfo(fetch(moshi_weights, names["moshi"]), fetch(mimi_weights, names["mimi"]),
                              fetch(tokenizer, names["tok"]), lm_config, raw, mimi_cfg, lm_gen_config=gen_cfg)

    def get_mimi(self, device: torch.device | str = "cuda") -> MimiModel:
        if self.lm_config is None:
            num_codebooks = 8
        else:
            num_codebooks = max(self.lm_config["dep_q"], self.lm_config["n_q"] - self.lm_config["dep_q"])
        return get_mimi(self.mimi_weights, self.mimi_config, num_codebooks=num_codebooks, device=device)

    def get_moshi(self, device: torch.device | str = "cuda", dtype: torch.dtype = torch.bfloat16,
                  load_weight: bool = True, **kwargs) -> LMModel:
        return get_moshi_lm(self.moshi_weights if load_weight else None, lm_kwargs=self.lm_config,
                            device=device, dtype=dtype, **kwargs)

    def get_text_tokenizer(self):
        import sentencepiece
        return sentencepiece.SentencePieceProcessor(str(self.tokenizer))
