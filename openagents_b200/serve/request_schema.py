"""Type and range checks for the JSON bodies of the HTTP routes.

Every field a route reads is checked here before anything is queued on the engine, so a mistyped request gets a
``400 invalid_request_error`` that names the field instead of an engine error, a dropped connection, or (worst) an exception
on the scheduling thread that every other request waits on.  Unknown fields are ignored, as OpenAI-compatible servers do.
"""
from __future__ import annotations

import math

MAX_STOP_STRINGS = 16
MAX_SEED = 2 ** 63 - 1
# names the chat template is always rendered with: a request may add variables (reasoning_effort, ...), not replace these
RESERVED_TEMPLATE_NAMES = frozenset({"messages", "template", "bos_token", "eos_token", "tools", "add_generation_prompt"})


class BadRequest(ValueError):
    """A request field of the wrong type or out of range; the message names the field."""


def _is_int(v) -> bool:
    return (isinstance(v, int) and not isinstance(v, bool)) or (isinstance(v, float) and math.isfinite(v) and v == int(v))


def _is_num(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool) and math.isfinite(v)


def integer(body: dict, key: str, lo: int | None = None, hi: int | None = None) -> int | None:
    """``body[key]`` as an int (a float with an integral value is accepted), None when absent or null."""
    v = body.get(key)
    if v is None:
        return None
    if not _is_int(v):
        raise BadRequest(f"{key} must be an integer")
    v = int(v)
    if (lo is not None and v < lo) or (hi is not None and v > hi):
        raise BadRequest(f"{key} must be " + (f"between {lo} and {hi}" if lo is not None and hi is not None else
                                              f"at least {lo}" if lo is not None else f"at most {hi}"))
    return v


def number(body: dict, key: str, lo: float | None = None, hi: float | None = None) -> float | None:
    v = body.get(key)
    if v is None:
        return None
    if not _is_num(v):
        raise BadRequest(f"{key} must be a finite number")
    if (lo is not None and v < lo) or (hi is not None and v > hi):
        raise BadRequest(f"{key} must be " + (f"between {lo} and {hi}" if lo is not None and hi is not None else
                                              f"at least {lo}" if lo is not None else f"at most {hi}"))
    return float(v)


def boolean(body: dict, key: str) -> bool:
    v = body.get(key)
    if v is None:
        return False
    if not isinstance(v, bool):
        raise BadRequest(f"{key} must be true or false")
    return v


def string(body: dict, key: str) -> str | None:
    v = body.get(key)
    if v is not None and not isinstance(v, str):
        raise BadRequest(f"{key} must be a string")
    return v


def stop_strings(body: dict) -> tuple[str, ...]:
    v = body.get("stop")
    if v is None or v == "" or v == []:
        return ()
    if isinstance(v, str):
        return (v,)
    if isinstance(v, list) and len(v) <= MAX_STOP_STRINGS and all(isinstance(s, str) for s in v):
        return tuple(s for s in v if s)
    raise BadRequest(f"stop must be a string or a list of at most {MAX_STOP_STRINGS} strings")


def sampling_fields(body: dict, default_max_tokens: int = 128, max_tokens: int | None = None) -> dict:
    """The sampling options of a request, checked.  ``max_tokens`` (alias ``max_output_tokens``) absent, null or 0 means the
    default, ``top_p`` 0 or null means 1 (no nucleus cut), ``top_k`` 0 means no cut: the conventions the routes have always had.
    ``max_tokens`` given as an argument overrides the body (the text-completion route has its own rule for 0)."""
    if max_tokens is None:
        max_tokens = integer(body, "max_tokens", 0) or integer(body, "max_output_tokens", 0) or default_max_tokens
    return {"max_tokens": max_tokens, "temperature": number(body, "temperature", 0.0) or 0.0,
            "top_p": number(body, "top_p", 0.0, 1.0) or 1.0, "top_k": integer(body, "top_k", 0, 2 ** 31 - 1) or 0,
            "stop": stop_strings(body), "seed": integer(body, "seed", 0, MAX_SEED)}


def sampling_params(body: dict, default_max_tokens: int = 128, max_tokens: int | None = None):
    """``sampling_fields`` as the scheduler's ``SamplingParams`` (imported here, so that this module stays importable without
    the engine: the gateway applies the same checks in a process that never loads a model)."""
    from .generation import SamplingParams
    return SamplingParams(**sampling_fields(body, default_max_tokens, max_tokens))


def messages(v, key: str = "messages") -> list[dict]:
    """A non-empty list of ``{"role": str, "content": str | list | null, ...}`` objects."""
    if not isinstance(v, list) or not v:
        raise BadRequest(f"{key} must be a non-empty list")
    for i, m in enumerate(v):
        if not isinstance(m, dict):
            raise BadRequest(f"{key}[{i}] must be an object")
        if not isinstance(m.get("role"), str) or not m["role"]:
            raise BadRequest(f"{key}[{i}].role must be a non-empty string")
        if not isinstance(m.get("content"), (str, list, type(None))):
            raise BadRequest(f"{key}[{i}].content must be a string, a list of parts or null")
        if not isinstance(m.get("tool_calls"), (list, type(None))):
            raise BadRequest(f"{key}[{i}].tool_calls must be a list")
    return v


def tools(body: dict) -> list[dict]:
    v = body.get("tools")
    if v is None:
        return []
    if not isinstance(v, list) or not all(isinstance(t, dict) for t in v):
        raise BadRequest("tools must be a list of objects")
    for i, t in enumerate(v):
        fn = t.get("function")
        if t.get("type", "function") != "function" or not isinstance(fn, dict) or not isinstance(fn.get("name"), str) or not fn["name"]:
            raise BadRequest(f"tools[{i}] must be {{\"type\": \"function\", \"function\": {{\"name\": ..., \"parameters\": ...}}}}")
        if not isinstance(fn.get("parameters"), (dict, type(None))) or not isinstance(fn.get("description"), (str, type(None))):
            raise BadRequest(f"tools[{i}].function: parameters must be an object and description a string")
    return v


def template_kwargs(body: dict) -> dict:
    v = body.get("chat_template_kwargs")
    if v is None:
        return {}
    if not isinstance(v, dict) or not all(isinstance(k, str) for k in v):
        raise BadRequest("chat_template_kwargs must be an object")
    clash = sorted(RESERVED_TEMPLATE_NAMES & set(v))
    if clash:
        raise BadRequest(f"chat_template_kwargs may not set {', '.join(clash)}")
    return v


def common(body: dict) -> None:
    """Checks shared by every generating route; raises ``BadRequest``."""
    string(body, "model")
    sampling_fields(body)
    boolean(body, "stream")
    tools(body)
    template_kwargs(body)
    string(body, "previous_response_id")
    string(body, "user")
    string(body, "demand_kind")
    if not isinstance(body.get("logprobs"), (bool, int, type(None))):
        raise BadRequest("logprobs must be true, false or an integer")
    integer(body, "top_logprobs", 0)
    if body.get("messages") is not None:
        messages(body["messages"])
