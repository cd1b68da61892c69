"""Whole-model post-training ternarisation on the GPU — counterpart of the reference's
``t81.convert`` (t81/convert.py:100-264, metadata helpers :267-352).

``convert`` walks a model, swaps every ``nn.Linear`` for ``t81lib_b200.nn.Linear`` and — unlike
the reference, which copies the float weight and leaves quantisation to the first forward on the
CPU — quantises and packs each weight at once with the device kernel, where the weight already
lives.  A layer costs one kernel launch (a 4096 x 4096 weight packs in about 20 microseconds), so
a multi-billion-parameter model converts in well under a second of GPU time instead of hours of
Python loops.

Kept from the reference: the ``threshold`` / ``keep_biases_bf16`` arguments and their meaning,
``inplace=True`` for an instantiated model, the statistics line, the ``_t81_*`` attributes attached
to the model, and the ``t81_metadata.json`` side file written by ``save_pretrained_t81`` and read
back by ``from_pretrained_t81``.  Loading by name goes through ``transformers`` exactly as the
reference does and needs that package; converting an ``nn.Module`` instance does not.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Mapping, Optional

import torch
from torch import nn

from .nn import Linear as TernaryLinear
from . import torch as t81_torch

_METADATA_FILENAME = "t81_metadata.json"


@dataclass
class ConversionStats:
    """Bytes before and after, as t81/convert.py:31-35 counts them, plus what was done on the device."""
    float_bytes: int = 0
    ternary_bytes: int = 0
    replaced: int = 0
    packed_on_device: int = 0


def _ternary_byte_count(shape) -> int:
    rows, cols = shape
    return rows * ((cols + 47) // 48) * 16


def _convert_linear_layer(linear: nn.Module, threshold: float, keep_biases_bf16: bool, rule: str,
                          pack_now: bool, release_float: bool, stats: ConversionStats) -> Optional[nn.Module]:
    """t81/convert.py:100-139.  Returns the replacement, or None when ``linear`` is left as it is."""
    if isinstance(linear, TernaryLinear):
        linear.ternary_threshold = threshold
        linear.ternary_weight = None  # re-quantised with the new threshold on the next eval forward
        return None
    if not isinstance(linear, nn.Linear):
        return None
    weight = linear.weight
    ternary = TernaryLinear(linear.in_features, linear.out_features, bias=linear.bias is not None, device="meta",
                            dtype=weight.dtype, threshold=threshold, rule=rule)
    # the new module takes over the existing parameters: no second copy of the weights is made
    ternary.weight = linear.weight
    if linear.bias is not None:
        bias = linear.bias
        if not keep_biases_bf16 and bias.dtype == torch.bfloat16:
            bias = nn.Parameter(bias.detach().to(torch.float32), requires_grad=bias.requires_grad)
        ternary.bias = bias
    ternary.train(linear.training)
    stats.float_bytes += weight.numel() * weight.element_size()
    stats.ternary_bytes += _ternary_byte_count(tuple(weight.shape))
    stats.replaced += 1
    if pack_now and weight.is_cuda and not weight.is_meta:
        ternary.ternary_weight = t81_torch.TernaryTensor.from_float(weight.detach(), threshold=threshold, rule=rule)
        ternary.ternary_weight._float_source = None  # the module owns the float weight; do not pin a second reference
        if t81_torch.DECODE_STREAM_LAYOUT:
            # the decode-stream copy too (0.25 byte per weight), so that the first decode step — possibly inside a
            # CUDA graph capture — does not have to make it
            from . import ops
            tw = ternary.ternary_weight
            tw._t2 = ops.pack_t2(tw.packed, tw._rows, tw._k_actual)
        stats.packed_on_device += 1
        if release_float:
            # inference-only deployment: the packed bytes (2.67 bits per weight) replace the float weight
            ternary.weight = nn.Parameter(torch.empty(0, dtype=weight.dtype, device=weight.device), requires_grad=False)
            ternary._t81_float_released = True
            ternary.eval()
    return ternary


def _walk_and_replace(module: nn.Module, threshold: float, keep_biases_bf16: bool, rule: str, pack_now: bool,
                      release_float: bool, stats: ConversionStats) -> None:
    """t81/convert.py:142-153."""
    for name, child in list(module.named_children()):
        replacement = _convert_linear_layer(child, threshold, keep_biases_bf16, rule, pack_now, release_float, stats)
        if replacement is not None:
            setattr(module, name, replacement)
        else:
            _walk_and_replace(child, threshold, keep_biases_bf16, rule, pack_now, release_float, stats)


def _report_stats(stats: ConversionStats) -> None:
    """t81/convert.py:164-177."""
    if stats.ternary_bytes == 0:
        return
    mib = 1024 ** 2
    ratio = stats.float_bytes / stats.ternary_bytes
    print(f"t81.convert: replaced {stats.replaced} nn.Linear modules, "
          f"compressed {stats.float_bytes / mib:.2f} MiB -> {stats.ternary_bytes / mib:.2f} MiB "
          f"(ratio {ratio:.2f}), estimated VRAM savings {(stats.float_bytes - stats.ternary_bytes) / mib:.2f} MiB; "
          f"{stats.packed_on_device} packed on the device")


def _load_model(model_id_or_path: str, device_map, torch_dtype):
    """t81/convert.py:180-211: the first AutoModel class that accepts the checkpoint."""
    import transformers
    kwargs: dict = {"trust_remote_code": True, "device_map": device_map, "low_cpu_mem_usage": True}
    if torch_dtype is not None:
        kwargs["torch_dtype"] = torch_dtype
    classes = [getattr(transformers, n) for n in (
        "AutoModelForCausalLM", "AutoModelForSeq2SeqLM", "AutoModelForMaskedLM", "AutoModelForSequenceClassification",
        "AutoModelForTokenClassification", "AutoModelForQuestionAnswering", "AutoModelForMultipleChoice", "AutoModel")]
    last_error: Optional[Exception] = None
    for cls in classes:
        try:
            return cls.from_pretrained(model_id_or_path, **kwargs)
        except Exception as exc:  # the next class may fit the checkpoint
            last_error = exc
    raise last_error if last_error is not None else RuntimeError("Unable to instantiate model")


def convert_module(model: nn.Module, threshold: float = 0.45, keep_biases_bf16: bool = True, *, rule: str = "fixed",
                   pack_now: bool = True, release_float: bool = False, verbose: bool = True) -> ConversionStats:
    """Ternarise every ``nn.Linear`` below ``model`` in place (t81/convert.py:214-221) and return the
    statistics.  With ``pack_now`` weights that live on a CUDA device are quantised and packed there
    immediately; others are packed lazily by the first eval forward, like the reference.  ``release_float``
    drops the float weight of every layer packed here (inference only: such a layer cannot train, and its
    ``state_dict`` no longer holds the float weight)."""
    stats = ConversionStats()
    _walk_and_replace(model, threshold, keep_biases_bf16, rule, pack_now, release_float, stats)
    setattr(model, "_t81_threshold", threshold)
    setattr(model, "_t81_keep_biases_bf16", keep_biases_bf16)
    setattr(model, "_t81_rule", rule)
    setattr(model, "_t81_compression_stats", stats)
    if verbose:
        _report_stats(stats)
    return stats


def convert(model_id_or_path, threshold: float = 0.45, keep_biases_bf16: bool = True,
            device_map: "str | Mapping[str, Any] | None" = "auto", torch_dtype: Optional[torch.dtype] = None, *,
            inplace: bool = False, force_cpu_device_map: bool = False, rule: str = "fixed", pack_now: bool = True,
            release_float: bool = False) -> nn.Module:
    """t81/convert.py:224-264.  A checkpoint name or path is loaded through ``transformers``; a model instance
    is converted as it is and, as in the reference, needs ``inplace=True``."""
    if isinstance(model_id_or_path, nn.Module):
        if not inplace:
            raise ValueError("convert() requires inplace=True when passing a PreTrainedModel instance")
        model = model_id_or_path
        effective_device_map = None
    else:
        effective_device_map = None if force_cpu_device_map else device_map
        if isinstance(effective_device_map, str) and effective_device_map.strip().lower() == "none":
            effective_device_map = None
        model = _load_model(str(model_id_or_path), effective_device_map, torch_dtype)
    convert_module(model, threshold, keep_biases_bf16, rule=rule, pack_now=pack_now, release_float=release_float)
    spec: dict = {"device_map": effective_device_map, "torch_dtype": torch_dtype, "threshold": threshold,
                  "keep_biases_bf16": keep_biases_bf16, "rule": rule}
    if isinstance(model_id_or_path, (str, Path)):
        spec["model_id_or_path"] = str(model_id_or_path)
    else:
        name = getattr(getattr(model, "config", None), "_name_or_path", None)
        if name is not None:
            spec["model_id_or_path"] = name
    setattr(model, "_t81_source_spec", spec)
    return model


def _metadata_path(directory: Path) -> Path:
    return directory / _METADATA_FILENAME


def save_pretrained_t81(model: nn.Module, save_directory, *, threshold: Optional[float] = None,
                        keep_biases_bf16: Optional[bool] = None, call_save_pretrained: bool = True,
                        save_fn: Optional[Callable[[nn.Module, Path], None]] = None, **kwargs: Any) -> None:
    """t81/convert.py:271-318: the model's own ``save_pretrained`` (or ``save_fn``) plus ``t81_metadata.json``.
    The float weights are what is saved, as in the reference; the packed form is rebuilt on load."""
    directory = Path(save_directory)
    directory.mkdir(parents=True, exist_ok=True)
    if call_save_pretrained:
        if any(getattr(m, "_t81_float_released", False) for m in model.modules()):
            raise RuntimeError("float weights were released at conversion (release_float=True); nothing to save")
        saver = save_fn or getattr(type(model), "__t81_original_save_pretrained__", None)
        if saver is not None:
            saver(model, directory, **kwargs)
        elif hasattr(model, "save_pretrained"):
            model.save_pretrained(directory, **kwargs)
        else:
            torch.save(model.state_dict(), directory / "pytorch_model.bin")
    metadata = {
        "threshold": threshold if threshold is not None else getattr(model, "_t81_threshold", 0.45),
        "keep_biases_bf16": keep_biases_bf16 if keep_biases_bf16 is not None else getattr(model, "_t81_keep_biases_bf16", True),
        "rule": getattr(model, "_t81_rule", "fixed"),
    }
    with _metadata_path(directory).open("w", encoding="utf-8") as handle:
        json.dump(metadata, handle)


def read_metadata(directory) -> dict:
    path = _metadata_path(Path(directory))
    if not path.exists():
        return {}
    with path.open("r", encoding="utf-8") as handle:
        return json.load(handle)


def from_pretrained_t81(cls, pretrained_model_name_or_path, *model_args: Any, threshold: Optional[float] = None,
                        keep_biases_bf16: Optional[bool] = None, device_map="auto", torch_dtype=None,
                        trust_remote_code: bool = True, loader: Optional[Callable[..., nn.Module]] = None,
                        **model_kwargs: Any) -> nn.Module:
    """t81/convert.py:321-352: read ``t81_metadata.json`` if present, load with ``cls.from_pretrained`` (or
    ``loader``), convert with the stored threshold, bias policy and rule."""
    metadata = read_metadata(pretrained_model_name_or_path)
    threshold = threshold if threshold is not None else metadata.get("threshold", 0.45)
    keep_biases_bf16 = keep_biases_bf16 if keep_biases_bf16 is not None else metadata.get("keep_biases_bf16", True)
    if loader is not None:
        model = loader(pretrained_model_name_or_path, *model_args, **model_kwargs)
    else:
        model = cls.from_pretrained(pretrained_model_name_or_path, *model_args, trust_remote_code=trust_remote_code,
                                    device_map=device_map, torch_dtype=torch_dtype, **model_kwargs)
    convert_module(model, threshold, keep_biases_bf16, rule=metadata.get("rule", "fixed"), verbose=False)
    return model


__all__ = ["convert", "convert_module", "save_pretrained_t81", "from_pretrained_t81", "read_metadata", "ConversionStats"]
