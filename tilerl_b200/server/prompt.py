"""Chat template, sampling defaults, think-splitting, tool rendering and parsing.

* ChatML rendering with optional ``<think>`` pre-fill (thinking on: the assistant turn
  opens with ``<think>\\n``; off: an empty think block is pre-filled so the model answers
  directly).
* Model-card sampling defaults (thinking: T=1.0 / top_p .95 / top_k 20; non-thinking:
  .7 / .8 / 20); top-k always comes from here, never from the request.
* ``reasoning_effort`` maps to a cap on think tokens (the engine forces ``</think>``).
* Tools are rendered into the system turn; calls come back as
  ``<tool_call><function=name><parameter=k>v</parameter></function></tool_call>`` XML and
  are parsed into typed arguments using the tool's JSON schema.
* Unknown request fields are refused (400), not silently ignored.

Parity: reference ``src/tilerl/prompt.py`` -- ``SAMPLING:15``, ``render_chat:19``,
``sampling:64``, ``split_think:146``, ``render_tools:194``, ``EFFORT_CAPS:292``,
``await_completion:367``; tool-call parsing ``src/tilerl/messages.py:139``.
"""
from __future__ import annotations

import asyncio
import json
import re
import time
from typing import Any, Dict, Iterable, List, Optional, Tuple

SAMPLING = {
    True: dict(temperature=1.0, top_p=0.95, top_k=20),    # thinking
    False: dict(temperature=0.7, top_p=0.8, top_k=20),    # non-thinking
}
EFFORT_CAPS = {"none": 0, "minimal": 64, "low": 512, "medium": 2048, "high": 8192}


class BadRequest(ValueError):
    """Maps to HTTP 400 with an OpenAI-style error body."""

    def __init__(self, message: str, param: Optional[str] = None):
        super().__init__(message)
        self.param = param


def unknown_fields(body: Dict[str, Any], allowed: Iterable[str]) -> List[str]:
    allowed = set(allowed)
    return sorted(k for k in body if k not in allowed)


def refuse_unknown(body: Dict[str, Any], allowed: Iterable[str]) -> None:
    bad = unknown_fields(body, allowed)
    if bad:
        raise BadRequest(f"unsupported field(s): {', '.join(bad)}", bad[0])


def content_text(content: Any) -> str:
    """OpenAI/Anthropic message content: a string or a list of typed parts."""
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    out = []
    for part in content:
        if isinstance(part, str):
            out.append(part)
        elif part.get("type") in ("text", "input_text", "output_text"):
            out.append(part.get("text", ""))
        elif part.get("type") == "tool_result":
            out.append(content_text(part.get("content")))
        elif part.get("type") in ("image_url", "image", "input_image"):
            raise BadRequest("image content is not supported by this model", "messages")
    return "".join(out)


def render_tools(tools: Optional[List[Dict[str, Any]]]) -> str:
    if not tools:
        return ""
    lines = ["# Tools", "", "You may call one or more functions to assist with the user query.",
             "Function signatures are given inside <tools></tools>:", "<tools>"]
    for t in tools:
        fn = t.get("function", t)
        lines.append(json.dumps({"name": fn["name"], "description": fn.get("description", ""),
                                 "parameters": fn.get("parameters", fn.get("input_schema", {}))},
                                ensure_ascii=False))
    lines += ["</tools>", "",
              "To call a function reply with:", "<tool_call>", "<function=NAME>",
              "<parameter=ARG>", "value", "</parameter>", "</function>", "</tool_call>"]
    return "\n".join(lines)


def render_tool_call(name: str, args: Dict[str, Any]) -> str:
    parts = [f"<tool_call>\n<function={name}>"]
    for k, v in args.items():
        parts.append(f"<parameter={k}>\n{v if isinstance(v, str) else json.dumps(v)}\n</parameter>")
    parts.append("</function>\n</tool_call>")
    return "\n".join(parts)


def render_chat(messages: List[Dict[str, Any]], *, tools=None, enable_thinking: bool = True,
                add_generation_prompt: bool = True) -> str:
    out: List[str] = []
    system = ""
    rest = list(messages)
    if rest and rest[0].get("role") in ("system", "developer"):
        system = content_text(rest.pop(0).get("content"))
    tool_text = render_tools(tools)
    if system or tool_text:
        out.append("<|im_start|>system\n" + "\n\n".join(x for x in (system, tool_text) if x) + "<|im_end|>\n")
    for m in rest:
        role = m.get("role")
        text = content_text(m.get("content"))
        if role == "assistant":
            for tc in m.get("tool_calls") or []:
                fn = tc.get("function", tc)
                args = fn.get("arguments", {})
                if isinstance(args, str):
                    try:
                        args = json.loads(args or "{}")
                    except json.JSONDecodeError:
                        args = {"arguments": args}
                text += ("\n" if text else "") + render_tool_call(fn["name"], args)
            out.append(f"<|im_start|>assistant\n{text}<|im_end|>\n")
        elif role == "tool":
            out.append(f"<|im_start|>user\n<tool_response>\n{text}\n</tool_response><|im_end|>\n")
        elif role in ("user", "system", "developer"):
            out.append(f"<|im_start|>{'system' if role != 'user' else 'user'}\n{text}<|im_end|>\n")
        else:
            raise BadRequest(f"unknown message role {role!r}", "messages")
    if add_generation_prompt:
        out.append("<|im_start|>assistant\n" + ("<think>\n" if enable_thinking else "<think>\n\n</think>\n\n"))
    return "".join(out)


def sampling(body: Dict[str, Any], thinking: bool) -> Dict[str, Any]:
    """Request fields over model-card defaults (``top_k`` is an extension the web client sends;
    0 switches the restriction off)."""
    d = dict(SAMPLING[bool(thinking)])
    for k in ("temperature", "top_p"):
        if body.get(k) is not None:
            d[k] = float(body[k])
    if body.get("top_k") is not None:
        try:
            d["top_k"] = int(body["top_k"])
        except (TypeError, ValueError):
            raise BadRequest("top_k must be an integer", "top_k") from None
        if d["top_k"] < 0:
            raise BadRequest("top_k must be >= 0", "top_k")
    if not 0.0 <= d["temperature"] <= 2.0:
        raise BadRequest("temperature must be in [0, 2]", "temperature")
    if not 0.0 < d["top_p"] <= 1.0:
        raise BadRequest("top_p must be in (0, 1]", "top_p")
    return d


def think_cap(effort: Optional[str], budget_tokens: Optional[int] = None) -> Optional[int]:
    if budget_tokens is not None:
        return max(0, int(budget_tokens))
    if effort is None:
        return None
    if effort not in EFFORT_CAPS:
        raise BadRequest(f"reasoning_effort must be one of {sorted(EFFORT_CAPS)}", "reasoning_effort")
    return EFFORT_CAPS[effort]


def split_think(text: str, thinking: bool) -> Tuple[str, str]:
    """(reasoning, answer).  With thinking on, the prompt already opened ``<think>``, so
    everything up to the first ``</think>`` is reasoning."""
    if "</think>" in text:
        head, tail = text.split("</think>", 1)
        return head.replace("<think>", "").strip("\n"), tail.lstrip("\n")
    if thinking:
        return text.replace("<think>", "").strip("\n"), ""
    return "", text


_TOOL_RE = re.compile(r"<tool_call>\s*<function=([^>\s]+)>(.*?)</function>\s*</tool_call>", re.S)
_PARAM_RE = re.compile(r"<parameter=([^>\s]+)>\n?(.*?)\n?</parameter>", re.S)


def _coerce(value: str, schema: Optional[Dict[str, Any]]) -> Any:
    t = (schema or {}).get("type")
    if t in ("integer", "number", "boolean", "object", "array", "null"):
        try:
            v = json.loads(value)
            if t == "integer" and isinstance(v, float) and v.is_integer():
                v = int(v)
            return v
        except json.JSONDecodeError:
            return value
    return value


def parse_tool_calls(text: str, tools: Optional[List[Dict[str, Any]]] = None) -> Tuple[str, List[Dict[str, Any]]]:
    """Strip tool-call XML from ``text``; return (remaining text, [{name, arguments}])."""
    schemas = {}
    for t in tools or []:
        fn = t.get("function", t)
        schemas[fn["name"]] = (fn.get("parameters") or fn.get("input_schema") or {}).get("properties", {})
    calls = []
    for m in _TOOL_RE.finditer(text):
        name, body = m.group(1), m.group(2)
        props = schemas.get(name, {})
        args = {k: _coerce(v, props.get(k)) for k, v in _PARAM_RE.findall(body)}
        calls.append({"name": name, "arguments": args})
    return _TOOL_RE.sub("", text).strip(), calls


def holdback(text: str, markers: Iterable[str]) -> int:
    """How many trailing characters of ``text`` might be the start of a marker (stop string
    or tool-call tag) and so must not be streamed yet."""
    keep = 0
    for mk in markers:
        for n in range(min(len(mk) - 1, len(text)), 0, -1):
            if text.endswith(mk[:n]):
                keep = max(keep, n)
                break
    return keep


async def await_completion(engine, rid: int, *, poll_s: float = 0.02, timeout_s: Optional[float] = None):
    """Poll ``engine.take`` until the request finishes; cancel it on timeout."""
    t0 = time.monotonic()
    while True:
        res = engine.take(rid)
        if res is not None:
            return res
        if timeout_s is not None and time.monotonic() - t0 > timeout_s:
            engine.cancel(rid)
            raise TimeoutError(f"completion exceeded {timeout_s}s")
        await asyncio.sleep(poll_s)
