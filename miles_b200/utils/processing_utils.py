"""Tokenizer / processor loading and prompt encoding shared by the data source, the reward hub and the servers.

``load_tokenizer`` and ``load_processor`` wrap the Hugging Face loaders (a model without a processor simply has
none: text-only). ``apply_chat_template`` renders messages (with tools) and returns text or ids; ``encode_multimodal``
runs a processor over text plus images and returns the token ids together with the extra model inputs, so that a
sample can carry them to the trainer.

Reference counterpart: miles/utils/processing_utils.py (192 lines).
"""
from __future__ import annotations

import base64
import io
from typing import Any, Optional, Sequence


def load_tokenizer(name_or_path: str, trust_remote_code: bool = True, **kw) -> Any:
    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(name_or_path, trust_remote_code=trust_remote_code, **kw)
    if getattr(tok, "pad_token_id", None) is None and getattr(tok, "eos_token_id", None) is not None:
        tok.pad_token_id = tok.eos_token_id
    return tok


def load_processor(name_or_path: str, trust_remote_code: bool = True, **kw) -> Optional[Any]:
    """The multimodal processor of a checkpoint, or None for a text-only model."""
    try:
        from transformers import AutoProcessor

        proc = AutoProcessor.from_pretrained(name_or_path, trust_remote_code=trust_remote_code, **kw)
    except Exception:
        return None
    # AutoProcessor falls back to the plain tokenizer for text-only checkpoints
    return proc if hasattr(proc, "image_processor") or hasattr(proc, "feature_extractor") else None


def apply_chat_template(tokenizer: Any, messages: Sequence[dict], tools: Optional[Sequence[dict]] = None,
                        add_generation_prompt: bool = True, tokenize: bool = False, **template_kwargs):
    kw = dict(template_kwargs)
    if tools:
        kw["tools"] = list(tools)
    return tokenizer.apply_chat_template(list(messages), tokenize=tokenize, add_generation_prompt=add_generation_prompt, **kw)


def decode_image(item: Any):
    """An image given as a PIL image, a path, raw bytes or a base64 / data-URL string."""
    from PIL import Image

    if hasattr(item, "size") and hasattr(item, "mode"):
        return item
    if isinstance(item, (bytes, bytearray)):
        return Image.open(io.BytesIO(item)).convert("RGB")
    if isinstance(item, str):
        if item.startswith("data:"):
            item = item.split(",", 1)[1]
            return Image.open(io.BytesIO(base64.b64decode(item))).convert("RGB")
        try:
            return Image.open(item).convert("RGB")
        except (FileNotFoundError, OSError):
            return Image.open(io.BytesIO(base64.b64decode(item))).convert("RGB")
    raise TypeError(f"cannot read an image from {type(item).__name__}")


def encode_multimodal(processor: Any, text: str, images: Optional[Sequence[Any]] = None) -> dict:
    """``{"input_ids": [...], "multimodal_inputs": {...}}`` — the ids the engine is fed and the tensors (pixel values,
    grids) that have to reach the trainer with the sample."""
    imgs = [decode_image(i) for i in (images or [])]
    out = processor(text=[text], images=imgs or None, return_tensors="pt")
    ids = out["input_ids"][0].tolist()
    extra = {k: v for k, v in out.items() if k not in ("input_ids", "attention_mask")}
    return {"input_ids": ids, "multimodal_inputs": extra}


def image_to_data_url(img: Any, fmt: str = "PNG") -> str:
    buf = io.BytesIO()
    decode_image(img).save(buf, format=fmt)
    return f"data:image/{fmt.lower()};base64," + base64.b64encode(buf.getvalue()).decode()
