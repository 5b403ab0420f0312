"""A dependency-free byte-level tokenizer with a chat template, for text environments, the HTTP server and tests when
no pretrained tokenizer files are available (there is no network here). Ids 0..255 are bytes; specials follow."""

from __future__ import annotations


def chat_ids(tokenizer, messages, add_generation_prompt: bool = True, **kw) -> list[int]:
    """Token ids of a conversation through the tokenizer's chat template. Tokenizers differ in what ``tokenize=True``
    returns (a list of ids; or, in recent ``transformers``, a mapping with ``input_ids``; possibly batched): this gives
    the flat list either way."""
    out = tokenizer.apply_chat_template(messages, add_generation_prompt=add_generation_prompt, tokenize=True, **kw)
    if hasattr(out, "keys") and "input_ids" in out:
        out = out["input_ids"]
    if hasattr(out, "tolist"):
        out = out.tolist()
    out = list(out)
    if out and isinstance(out[0], (list, tuple)):
        out = list(out[0])
    return [int(t) for t in out]


def chat_ids_continuation(tokenizer, messages, **kw) -> list[int]:
    """Ids of ``messages`` (environment observations, tool results) as they appear INSIDE a running conversation, ending
    with the generation prompt of the next assistant turn. Rendered alone, many templates would open with a preamble
    (a default system prompt, a begin-of-text token) that must not be repeated in mid-context: the messages are rendered
    after a fixed dummy turn whose ids are cut off again. A template that is not prefix-stable under that falls back to
    the stand-alone rendering (reference: skyrl/train/generators/utils.py ``encode_messages_subset``)."""
    base = [{"role": "user", "content": "."}]
    head = chat_ids(tokenizer, base, False, **kw)
    full = chat_ids(tokenizer, base + list(messages), True, **kw)
    if head and full[:len(head)] == head:
        return full[len(head):]
    return chat_ids(tokenizer, messages, True, **kw)


class ByteTokenizer:
    BOS, EOS, IM_START, IM_END, PAD = 256, 257, 258, 259, 260
    vocab_size = 261

    def __init__(self):
        self.eos_token_id, self.pad_token_id, self.bos_token_id = self.EOS, self.PAD, self.BOS

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        ids = list(text.encode("utf-8"))
        return ([self.BOS] + ids) if add_special_tokens else ids

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        out = bytearray()
        names = {self.BOS: "<s>", self.EOS: "</s>", self.IM_START: "<|im_start|>", self.IM_END: "<|im_end|>", self.PAD: ""}
        for t in ids:
            t = int(t)
            if t < 256:
                out.append(t)
            elif not skip_special_tokens:
                out += names.get(t, "").encode()
        return out.decode("utf-8", errors="replace")

    def encode_rendered(self, text: str) -> list[int]:
        """Text produced by ``apply_chat_template(tokenize=False)`` back to ids: the names of the special tokens become
        their ids again, everything else is bytes."""
        import re

        names = {"<s>": self.BOS, "</s>": self.EOS, "<|im_start|>": self.IM_START, "<|im_end|>": self.IM_END}
        ids: list[int] = []
        for piece in re.split("(" + "|".join(re.escape(n) for n in names) + ")", text):
            if piece in names:
                ids.append(names[piece])
            elif piece:
                ids += self.encode(piece)
        return ids

    def apply_chat_template(self, messages: list[dict], add_generation_prompt: bool = True, tokenize: bool = True, **_):
        ids: list[int] = []
        for m in messages:
            ids += [self.IM_START] + self.encode(f"{m['role']}\n{m['content']}") + [self.IM_END] + self.encode("\n")
        if add_generation_prompt:
            ids += [self.IM_START] + self.encode("assistant\n")
        return ids if tokenize else self.decode(ids, skip_special_tokens=False)
