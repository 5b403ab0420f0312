"""Function calling for models without a native tool-call channel: OpenAI-style tool schemas and ``tool_calls`` messages
to and from plain text (reference: skyrl-agent/skyrl_agent/functional/function_calling.py, the OpenHands text protocol).

On the wire a call is

    <function=NAME>
    <parameter=KEY>value</parameter>
    <parameter=OTHER>
    a value that
    spans lines
    </parameter>
    </function>

at the END of an assistant message (reasoning may stand in front of it, nothing behind it, one call per message), and a
tool's answer is a user message ``EXECUTION RESULT of [NAME]:\\n...``. Generation can stop at ``STOP_WORDS`` (``</function``
without the ``>``); ``close_call`` repairs such a cut.

* ``tools_prompt(tools)``                      the text appended to the system message: every tool with its parameters
                                               (type, required or optional, allowed values) and the calling format;
* ``parse_call(text, tools)``                  ``(text in front of the call, {"name", "arguments"} or None)``; arguments are
                                               validated against the schema and converted to its types; problems raise
                                               ``FunctionCallValidationError`` with a message fit to show the model;
* ``call_to_text(tool_call)``                  an OpenAI ``tool_calls`` entry as wire text;
* ``to_text_messages(messages, tools)``        a conversation with ``tool_calls`` / ``tool`` messages as plain messages;
* ``to_tool_messages(messages, tools)``        the inverse (call ids are generated; a result is tied to the call before it).
"""

from __future__ import annotations

import json
import re
import uuid

STOP_WORDS = ["</function"]
_CALL = re.compile(r"<function=([^>]+)>\n?(.*?)</function>", re.S)
_PARAM = re.compile(r"<parameter=([^>]+)>(.*?)</parameter>", re.S)
_RESULT = re.compile(r"EXECUTION RESULT of \[(.*?)\]:\n(.*)", re.S)


class FunctionCallConversionError(ValueError):
    """A message cannot be converted (malformed ``tool_calls``, a tool result without a call ...)."""


class FunctionCallValidationError(ValueError):
    """The model's call does not fit the tool's schema; the message is written for the model."""


FORMAT_HELP = """To call a function, end your reply with exactly one block of this shape and write nothing after it:

<function=the_function_name>
<parameter=first_parameter>a short value</parameter>
<parameter=second_parameter>
a longer value may
run over several lines
</parameter>
</function>

Rules:
- the block starts with <function= and ends with </function>;
- every required parameter must be present, and only parameters the function lists;
- one call per reply; explain your reasoning, if you want to, BEFORE the block;
- when no function fits, simply answer in plain text.
"""


def _fn(tool: dict) -> dict:
    if tool.get("type", "function") != "function" or "function" not in tool:
        raise FunctionCallConversionError(f"not a function tool: {tool}")
    return tool["function"]


def describe_tools(tools: list[dict]) -> str:
    out = []
    for i, tool in enumerate(tools, 1):
        fn = _fn(tool)
        lines = [f"---- BEGIN FUNCTION #{i}: {fn['name']} ----", f"Description: {fn.get('description', '')}"]
        props = (fn.get("parameters") or {}).get("properties") or {}
        if props:
            need = set((fn.get("parameters") or {}).get("required") or [])
            lines.append("Parameters:")
            for j, (name, info) in enumerate(props.items(), 1):
                desc = info.get("description", "No description provided")
                if "enum" in info:
                    desc += "\nAllowed values: [" + ", ".join(f"`{v}`" for v in info["enum"]) + "]"
                lines.append(f"  ({j}) {name} ({info.get('type', 'string')}, {'required' if name in need else 'optional'}): {desc}")
        else:
            lines.append("No parameters are required for this function.")
        lines.append(f"---- END FUNCTION #{i} ----")
        out.append("\n".join(lines))
    return "\n\n".join(out) + "\n"


def tools_prompt(tools: list[dict]) -> str:
    return "\nYou have access to the following functions:\n\n" + describe_tools(tools) + "\n" + FORMAT_HELP


def call_to_text(tool_call: dict) -> str:
    for key in ("function", "id", "type"):
        if key not in tool_call:
            raise FunctionCallConversionError(f"a tool call needs the key {key!r}")
    if tool_call["type"] != "function":
        raise FunctionCallConversionError("a tool call's type must be 'function'")
    args = tool_call["function"].get("arguments", {})
    if isinstance(args, str):
        try:
            args = json.loads(args or "{}")
        except json.JSONDecodeError as e:
            raise FunctionCallConversionError(f"the arguments are not JSON: {tool_call['function']['arguments']!r}") from e
    parts = [f"<function={tool_call['function']['name']}>"]
    for k, v in args.items():
        text = v if isinstance(v, str) else json.dumps(v)
        parts.append(f"<parameter={k}>\n{text}\n</parameter>" if "\n" in text else f"<parameter={k}>{text}</parameter>")
    return "\n".join(parts + ["</function>"])


def close_call(text: str) -> str:
    """Repair a message that generation cut at a stop word: ``...</function`` gets its ``>``; an open call whose last
    parameter was closed gets ``</function>``."""
    if "<function=" not in text:
        return text
    if text.rstrip().endswith("</function"):
        return text.rstrip() + ">"
    if "</function>" not in text[text.rfind("<function="):] and text.rstrip().endswith("</parameter>"):
        return text.rstrip() + "\n</function>"
    return text


def _convert(value: str, info: dict, fn_name: str, key: str):
    kind = info.get("type", "string")
    try:
        if kind == "integer":
            out = int(value)
        elif kind == "number":
            out = float(value)
        elif kind == "boolean":
            if value.strip().lower() not in ("true", "false"):
                raise ValueError
            out = value.strip().lower() == "true"
        elif kind in ("array", "object"):
            out = json.loads(value)
            if not isinstance(out, list if kind == "array" else dict):
                raise ValueError
        else:
            out = value
    except (ValueError, json.JSONDecodeError):
        raise FunctionCallValidationError(f"Parameter '{key}' of function '{fn_name}' must be of type {kind}, got: {value!r}") from None
    if "enum" in info and out not in info["enum"]:
        raise FunctionCallValidationError(f"Parameter '{key}' of function '{fn_name}' is {out!r}; allowed values: {info['enum']}")
    return out


def parse_call(text: str, tools: list[dict]) -> tuple[str, dict | None]:
    text = close_call(text)
    m = _CALL.search(text)
    if m is None:
        if "<function=" in text:
            raise FunctionCallValidationError("The function call is not closed: it must end with </function>.")
        return text, None
    name = m.group(1).strip()
    fn = next((f for f in map(_fn, tools) if f["name"] == name), None)
    if fn is None:
        raise FunctionCallValidationError(f"Function '{name}' is not available. Available functions: {[f['function']['name'] for f in tools]}")
    props = (fn.get("parameters") or {}).get("properties") or {}
    need = set((fn.get("parameters") or {}).get("required") or [])
    args: dict = {}
    for pm in _PARAM.finditer(m.group(2)):
        key, raw = pm.group(1).strip(), pm.group(2)
        if key in args:
            raise FunctionCallValidationError(f"Parameter '{key}' is given twice in the call of '{name}'.")
        if props and key not in props:
            raise FunctionCallValidationError(f"Parameter '{key}' is not accepted by function '{name}'. Allowed parameters: {sorted(props)}")
        raw = raw[1:] if raw.startswith("\n") else raw
        raw = raw[:-1] if raw.endswith("\n") else raw
        args[key] = _convert(raw, props.get(key, {}), name, key)
    missing = sorted(need - set(args))
    if missing:
        raise FunctionCallValidationError(f"Missing required parameters for function '{name}': {missing}")
    return text[:m.start()].rstrip(), {"name": name, "arguments": args}


def _text_of(content) -> str:
    if isinstance(content, str) or content is None:
        return content or ""
    return "".join(p.get("text", "") for p in content if isinstance(p, dict) and p.get("type") == "text")


def to_text_messages(messages: list[dict], tools: list[dict], add_tools_prompt: bool = True) -> list[dict]:
    out: list[dict] = []
    names: dict[str, str] = {}                         # tool_call_id -> function name
    seen_system = False
    for m in messages:
        role, text = m["role"], _text_of(m.get("content"))
        if role == "system":
            seen_system = True
            out.append({"role": "system", "content": text + (tools_prompt(tools) if add_tools_prompt else "")})
        elif role == "assistant":
            calls = m.get("tool_calls") or []
            if len(calls) > 1:
                raise FunctionCallConversionError("the text protocol carries one call per message")
            if calls:
                names[calls[0]["id"]] = calls[0]["function"]["name"]
                text = (text + "\n\n" if text else "") + call_to_text(calls[0])
            out.append({"role": "assistant", "content": text})
        elif role == "tool":
            name = m.get("name") or names.get(m.get("tool_call_id"))
            if name is None:
                raise FunctionCallConversionError("a tool message without a name and without a known tool_call_id")
            out.append({"role": "user", "content": f"EXECUTION RESULT of [{name}]:\n{text}"})
        else:
            out.append({"role": role, "content": text})
    if add_tools_prompt and not seen_system:
        out.insert(0, {"role": "system", "content": tools_prompt(tools).lstrip("\n")})
    return out


def to_tool_messages(messages: list[dict], tools: list[dict]) -> list[dict]:
    out: list[dict] = []
    pending: tuple[str, str] | None = None             # (call id, function name) that waits for its result
    suffix = tools_prompt(tools)
    for m in messages:
        role, text = m["role"], _text_of(m.get("content"))
        if role == "system":
            out.append({"role": "system", "content": text.replace(suffix, "")})
        elif role == "assistant":
            before, call = parse_call(text, tools)
            msg: dict = {"role": "assistant", "content": before}
            if call is not None:
                cid = "call_" + uuid.uuid4().hex[:12]
                msg["tool_calls"] = [{"id": cid, "type": "function", "function": {"name": call["name"], "arguments": json.dumps(call["arguments"])}}]
                pending = (cid, call["name"])
            out.append(msg)
        elif role == "user" and (r := _RESULT.match(text)) is not None:
            if pending is None or pending[1] != r.group(1):
                raise FunctionCallConversionError(f"an execution result of [{r.group(1)}] without a call of that function before it")
            out.append({"role": "tool", "tool_call_id": pending[0], "name": pending[1], "content": r.group(2)})
            pending = None
        else:
            out.append({"role": role, "content": text})
    return out
