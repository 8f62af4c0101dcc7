"""Tool calling for the model server and its client.

Server side: tool schemas are rendered into the prompt in a fixed, cache-friendly form; the model
answers with ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>`` blocks (any number in one
turn: parallel same-turn calls), which are parsed into OpenAI ``tool_calls``.  ``tool_choice`` may be
``auto``, ``none``, ``required`` or a named function; ``required`` / named with no parsed call is a
typed failure, not a silent text answer.  While streaming, text outside the blocks goes out as
``delta.content`` and each block as ``delta.tool_calls`` entries (name first, then the arguments).

Client side (the node runtime's attach-only client): assemble streamed ``delta.tool_calls`` fragments
by index back into whole calls, and run the tool loop (call the model, execute the requested tools,
append ``role: tool`` results, repeat until the model answers in text or the step limit is reached).

Reference: the serving surface is described in apps/pylon/docs/2026-06-09-pylon-qwen35-local-inference-roadmap.md:110-134,
343-386 (required / auto / parallel same-turn calls, streamed ``delta.tool_calls``); the client in
apps/pylon/packages/runtime/src/backends/psionic-qwen/client.ts:44-83; the provider-neutral request in
apps/pylon/packages/runtime/src/llm/request.ts:5-37 (generation options, tool choice auto / none /
required / named).
"""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field

from ..gateway.prompt_cache import serialize_tool_schemas

OPEN, CLOSE = "<tool_call>", "</tool_call>"
_BLOCK = re.compile(re.escape(OPEN) + r"\s*(\{.*?\})\s*" + re.escape(CLOSE), re.S)


class ToolCallError(Exception):
    def __init__(self, kind: str, message: str):
        super().__init__(message)
        self.kind = kind


def function_names(tools) -> set:
    """Names of the well-formed function tools in ``tools`` (entries of any other shape are ignored)."""
    if not isinstance(tools, (list, tuple)):
        return set()
    return {t["function"]["name"] for t in tools
            if isinstance(t, dict) and t.get("type", "function") == "function" and isinstance(t.get("function"), dict)
            and isinstance(t["function"].get("name"), str) and t["function"]["name"]}


def normalize_tool_choice(choice, tools) -> tuple[str, str | None]:
    """-> (mode, function name) with mode in auto | none | required | named."""
    names = function_names(tools)
    if choice is None:
        return ("auto" if names else "none"), None
    if isinstance(choice, str):
        if choice not in ("auto", "none", "required"):
            raise ToolCallError("invalid_tool_choice", f"tool_choice {choice!r} is not auto, none or required")
        if choice == "required" and not names:
            raise ToolCallError("invalid_tool_choice", "tool_choice required needs tools")
        return choice, None
    fn = choice.get("function") if isinstance(choice, dict) else None
    name = fn.get("name") if isinstance(fn, dict) else None
    if not isinstance(name, str) or name not in names:
        raise ToolCallError("invalid_tool_choice", f"tool_choice names an unknown function {name!r}")
    return "named", name


def render_tools_system_message(tools, mode: str, name: str | None) -> dict | None:
    """A stable system message (same tools -> same bytes) describing the tools and the call format."""
    if mode == "none" or not tools:
        return None
    rule = {"auto": "Call a tool only when it helps.", "required": "You must call at least one tool.",
            "named": f"You must call the tool {name}."}[mode]
    text = ("You can call tools. To call one, answer with " + OPEN + '{"name": <tool name>, "arguments": <JSON object>}' + CLOSE
            + " (one block per call; several blocks in one answer run in parallel). " + rule + "\nTools:\n" + serialize_tool_schemas(list(tools)))
    return {"role": "system", "content": text, "stable_kind": "toolSchemas"}


def parse_tool_calls(text: str, tools=None) -> tuple[str, list[dict]]:
    """-> (text outside the blocks, OpenAI tool_calls).  Malformed blocks and unknown names are dropped into the text."""
    names = function_names(tools) if tools is not None else None
    calls, out, pos = [], [], 0
    for m in _BLOCK.finditer(text):
        try:
            obj = json.loads(m.group(1))
            ok = isinstance(obj, dict) and isinstance(obj.get("name"), str) and isinstance(obj.get("arguments", {}), dict)
        except json.JSONDecodeError:
            ok = False
        if ok and (names is None or obj["name"] in names):
            out.append(text[pos:m.start()])
            pos = m.end()
            calls.append({"id": "call_" + uuid.uuid4().hex[:24], "type": "function",
                          "function": {"name": obj["name"], "arguments": json.dumps(obj.get("arguments", {}), separators=(",", ":"))}})
    out.append(text[pos:])
    return "".join(out).strip(), calls


def finish_with_tools(text: str, tools, mode: str, name: str | None) -> tuple[dict, str]:
    """-> (assistant message, finish_reason) for a completed generation."""
    if mode == "none":
        return {"role": "assistant", "content": text}, "stop"
    content, calls = parse_tool_calls(text, tools)
    if mode == "named":
        calls = [c for c in calls if c["function"]["name"] == name]
    if mode in ("required", "named") and not calls:
        raise ToolCallError("tool_call_required", "the model did not produce the required tool call")
    if not calls:
        return {"role": "assistant", "content": content}, "stop"
    return {"role": "assistant", "content": content or None, "tool_calls": calls}, "tool_calls"


class ToolCallStreamSplitter:
    """Feed generated text piece by piece; get back stream deltas: ``{"content": ...}`` for text outside tool-call
    blocks and ``{"tool_calls": [...]}`` for each completed block (first a delta with id and name, then one with
    the arguments), so that a client never sees half a block as content."""

    def __init__(self, tools=None):
        self.buf, self.n_calls, self.tools = "", 0, tools

    def feed(self, piece: str) -> list[dict]:
        self.buf += piece
        out = []
        while True:
            i = self.buf.find(OPEN)
            if i < 0:
                # keep a tail that could still become an opening tag
                keep = next((k for k in range(min(len(OPEN) - 1, len(self.buf)), 0, -1) if OPEN.startswith(self.buf[-k:])), 0)
                if len(self.buf) > keep:
                    out.append({"content": self.buf[: len(self.buf) - keep]})
                    self.buf = self.buf[len(self.buf) - keep:]
                return out
            if i > 0:
                out.append({"content": self.buf[:i]})
                self.buf = self.buf[i:]
            j = self.buf.find(CLOSE)
            if j < 0:
                return out
            block, self.buf = self.buf[: j + len(CLOSE)], self.buf[j + len(CLOSE):]
            _, calls = parse_tool_calls(block, self.tools)
            if not calls:
                out.append({"content": block})
                continue
            c = calls[0]
            out.append({"tool_calls": [{"index": self.n_calls, "id": c["id"], "type": "function", "function": {"name": c["function"]["name"], "arguments": ""}}]})
            out.append({"tool_calls": [{"index": self.n_calls, "function": {"arguments": c["function"]["arguments"]}}]})
            self.n_calls += 1

    def flush(self) -> list[dict]:
        out = [{"content": self.buf}] if self.buf else []
        self.buf = ""
        return out


# ---------------------------------------------------------------- client side
@dataclass
class GenerationOptions:
    max_tokens: int | None = None
    temperature: float | None = None
    top_p: float | None = None
    top_k: int | None = None
    stop: tuple = ()


@dataclass
class LlmRequest:
    """Provider-neutral request: what a backend lowers to its own wire format."""
    model: str
    messages: list
    system: str | None = None
    tools: list = field(default_factory=list)
    tool_choice: object = None            # "auto" | "none" | "required" | {"name": ...}
    options: GenerationOptions = field(default_factory=GenerationOptions)

    def to_openai(self, stream: bool = False) -> dict:
        msgs = ([{"role": "system", "content": self.system}] if self.system else []) + list(self.messages)
        body = {"model": self.model, "messages": msgs, "stream": stream}
        o = self.options
        for k, v in (("max_tokens", o.max_tokens), ("temperature", o.temperature), ("top_p", o.top_p), ("top_k", o.top_k)):
            if v is not None:
                body[k] = v
        if o.stop:
            body["stop"] = list(o.stop)
        if self.tools:
            body["tools"] = [{"type": "function", "function": t} if "function" not in t else t for t in self.tools]
            tc = self.tool_choice
            if tc is not None:
                body["tool_choice"] = {"type": "function", "function": {"name": tc["name"]}} if isinstance(tc, dict) else tc
        return body


class ToolCallDeltaAssembler:
    """Rebuild whole tool calls from streamed ``delta.tool_calls`` fragments (keyed by ``index``)."""

    def __init__(self):
        self.calls: dict[int, dict] = {}
        self.content = ""

    def feed(self, delta: dict):
        if isinstance(delta.get("content"), str):
            self.content += delta["content"]
        for frag in delta.get("tool_calls") or []:
            c = self.calls.setdefault(frag.get("index", 0), {"id": None, "type": "function", "function": {"name": "", "arguments": ""}})
            if frag.get("id"):
                c["id"] = frag["id"]
            fn = frag.get("function") or {}
            if fn.get("name"):
                c["function"]["name"] += fn["name"]
            if fn.get("arguments"):
                c["function"]["arguments"] += fn["arguments"]

    def result(self) -> list[dict]:
        return [self.calls[i] for i in sorted(self.calls)]


def parse_sse(lines) -> list[dict]:
    """``data: {...}`` lines of a chat-completions stream -> chunk objects (stops at ``[DONE]``)."""
    out = []
    for line in lines:
        line = line.decode() if isinstance(line, bytes) else line
        line = line.strip()
        if not line.startswith("data:"):
            continue
        payload = line[5:].strip()
        if payload == "[DONE]":
            break
        out.append(json.loads(payload))
    return out


def run_tool_loop(complete, request: LlmRequest, tool_impls: dict, max_steps: int = 8) -> dict:
    """``complete(openai_body) -> chat.completion object``.  Runs tools the model asks for until it answers in
    text.  Returns {"message", "steps", "transcript"}; an unknown tool or a tool exception becomes a tool
    message carrying the error, so the model can recover."""
    req = LlmRequest(request.model, list(request.messages), request.system, request.tools, request.tool_choice, request.options)
    for step in range(1, max_steps + 1):
        resp = complete(req.to_openai())
        msg = resp["choices"][0]["message"]
        req.messages.append(msg)
        calls = msg.get("tool_calls") or []
        if not calls:
            return {"message": msg, "steps": step, "transcript": req.messages}
        for c in calls:
            fn = c["function"]
            try:
                impl = tool_impls[fn["name"]]
                result = impl(**json.loads(fn["arguments"] or "{}"))
                content = result if isinstance(result, str) else json.dumps(result)
            except KeyError:
                content = json.dumps({"error": f"unknown tool {fn['name']}"})
            except Exception as e:      # tool failures are data for the model, not a crash of the loop
                content = json.dumps({"error": f"{type(e).__name__}: {e}"})
            req.messages.append({"role": "tool", "tool_call_id": c["id"], "content": content})
        if req.tool_choice in ("required",) or isinstance(req.tool_choice, dict):
            req.tool_choice = "auto"          # forcing a call on every step would never end
    raise ToolCallError("tool_loop_exhausted", f"no text answer after {max_steps} steps")
