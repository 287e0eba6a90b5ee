"""ChatML rendering through a Jinja2 template: prompt ids for inference, and training ids with an assistant-span
loss mask (from the assistant header through the closing ``<|im_end|>``), plus a parser for ``<tool_call>`` blocks
(reference ``loomformer.py:1459-1547``)."""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Tuple

from .tokenizers import special_id

_PKG_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


class ChatTemplate:
    def __init__(self, tok, template_path: str = "chat_template.jinja", template_source: Optional[str] = None) -> None:
        import jinja2
        self.tok = tok
        if template_source is None:
            path = template_path if os.path.isfile(template_path) else os.path.join(_PKG_ROOT, template_path)
            with open(path, "r", encoding="utf-8") as fh:
                template_source = fh.read()
        self.source = template_source
        self._tpl = jinja2.Environment().from_string(template_source)
        start, end = special_id(tok, "<|im_start|>"), special_id(tok, "<|im_end|>")
        if start is None or end is None:
            raise ValueError("ChatTemplate needs <|im_start|>/<|im_end|> in the tokenizer's vocab "
                             "(see data.tokenizers.SPECIAL_TOKENS) -- retrain it with those special tokens "
                             "if this one predates them.")
        self.im_start_id, self.im_end_id = start, end
        self.bos_id = special_id(tok, "<bos>")
        self.bos_token = "<bos>" if self.bos_id is not None else ""
        self.stop_ids = {i for i in (end, special_id(tok, "<eos>")) if i is not None}
        self._header = [start] + tok.encode("assistant\n")

    def render_text(self, messages: List[Dict], tools: Optional[List[Dict]] = None,
                    add_generation_prompt: bool = False) -> str:
        kw = {"messages": messages, "add_generation_prompt": add_generation_prompt, "bos_token": self.bos_token}
        if tools is not None:
            kw["tools"] = tools
        return self._tpl.render(**kw)

    def render_prompt_ids(self, messages: List[Dict], tools: Optional[List[Dict]] = None) -> List[int]:
        return self.tok.encode(self.render_text(messages, tools=tools, add_generation_prompt=True))

    def render_training_ids(self, messages: List[Dict], tools: Optional[List[Dict]] = None) -> Tuple[List[int], List[int]]:
        ids = self.tok.encode(self.render_text(messages, tools=tools))
        mask = [0] * len(ids)
        h, n, i = self._header, len(ids), 0
        while h and i <= n - len(h):
            if ids[i:i + len(h)] != h:
                i += 1
                continue
            j = i + len(h)
            k = j
            while k < n and ids[k] != self.im_end_id:
                k += 1
            for t in range(j, min(k, n - 1) + 1):
                mask[t] = 1
            i += len(h)
        return ids, mask

    @staticmethod
    def parse_tool_calls(text: str) -> List[Dict]:
        calls, pos = [], 0
        while True:
            s = text.find("<tool_call>", pos)
            e = text.find("</tool_call>", s) if s >= 0 else -1
            if s < 0 or e < 0:
                return calls
            pos = e + len("</tool_call>")
            try:
                obj = json.loads(text[s + len("<tool_call>"):e].strip())
            except Exception:
                continue
            calls.append({"id": f"call_{len(calls)}", "type": "function",
                          "function": {"name": obj.get("name"), "arguments": obj.get("arguments")}})
