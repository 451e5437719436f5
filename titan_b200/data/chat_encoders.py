"""Chat encoders: messages → (rendered text, token ids, assistant token ranges).

The assistant ranges ``[(start, end), ...]`` index the token sequence; only those tokens are supervised.

* `ChatMLEncoder` – renders with the tokenizer's chat template (ChatML when it has none) and finds the assistant
  replies by scanning for the ``<|im_start|>assistant\\n`` header up to the next end-of-turn / EOS token.
* `DSV4ChatEncoder` – DeepSeek-V4's own message format lives in an external ``encoding_dsv4.py`` (shipped with the
  checkpoint, not with this framework): the encoder loads that file, lets it merge tool messages, order tool results,
  drop or keep thinking blocks and render every message, then derives each assistant range from prefix tokenisations
  and checks that both prefixes are prefixes of the full tokenisation.

Parity: torchtitan_npu/patches/encoders/{base,dsv4}.py and the ChatML header scan of
patches/torchtitan/chat_dataset.py:238-262.
"""

from __future__ import annotations

import importlib.util
from typing import Any

from titan_b200.utils.logging import logger

__all__ = ["BaseChatEncoder", "ChatMLEncoder", "DSV4ChatEncoder", "build_chat_encoder", "chatml_assistant_ranges"]

AssistantRanges = list[tuple[int, int]]
VALID_THINKING_MODES = ("chat", "thinking")
VALID_REASONING_EFFORTS = ("max", "high")


class BaseChatEncoder:
    def encode_messages_with_assistant_ranges(self, messages: list[dict[str, Any]], tokenizer,
                                              eos_id: int) -> tuple[str, list[int], AssistantRanges]:
        raise NotImplementedError(f"{type(self).__name__}.encode_messages_with_assistant_ranges() not implemented")


def chatml_assistant_ranges(tokenizer, tokens: list[int], eos_id: int) -> AssistantRanges:
    header = tokenizer.encode("<|im_start|>assistant\n", add_bos=False, add_eos=False)
    end_turn = tokenizer.encode("<|im_end|>", add_bos=False, add_eos=False)
    stops = {eos_id} | ({end_turn[0]} if len(end_turn) == 1 else set())
    if not header:
        return []
    out, pos, n = [], 0, len(header)
    while pos < len(tokens):
        if tokens[pos: pos + n] == header:
            start = end = pos + n
            while end < len(tokens) and tokens[end] not in stops:
                end += 1
            out.append((start, min(end + 1, len(tokens))))  # the end-of-turn token is supervised too
            pos = end + 1
        else:
            pos += 1
    return out


class ChatMLEncoder(BaseChatEncoder):
    def encode_messages_with_assistant_ranges(self, messages, tokenizer, eos_id):
        text = tokenizer.apply_chat_template(messages, tokenize=False).rstrip("\n")
        tokens = tokenizer.encode(text, add_bos=True, add_eos=False)
        if not tokens or tokens[-1] != eos_id:
            tokens.append(eos_id)
        ranges = chatml_assistant_ranges(tokenizer, tokens, eos_id)
        if not ranges:
            raise ValueError("Unable to locate ChatML assistant ranges: the rendered text has no "
                             "'<|im_start|>assistant' header that the tokenizer encodes as such")
        return text, tokens, ranges


class DSV4ChatEncoder(BaseChatEncoder):
    def __init__(self, encoding_module_path: str, thinking_mode: str = "thinking", drop_thinking: bool = True,
                 reasoning_effort: str | None = None):
        if thinking_mode not in VALID_THINKING_MODES:
            raise ValueError(f"thinking_mode must be one of {VALID_THINKING_MODES}, got {thinking_mode!r}")
        if reasoning_effort is not None and reasoning_effort not in VALID_REASONING_EFFORTS:
            raise ValueError(f"reasoning_effort must be one of {VALID_REASONING_EFFORTS} or None, got "
                             f"{reasoning_effort!r}")
        spec = importlib.util.spec_from_file_location("encoding_dsv4", encoding_module_path)
        if spec is None or spec.loader is None:
            raise FileNotFoundError(f"Cannot load encoding module from: {encoding_module_path}")
        self._enc = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(self._enc)
        self.thinking_mode, self.drop_thinking, self.reasoning_effort = thinking_mode, drop_thinking, reasoning_effort
        logger.info("DSV4 chat encoder loaded from %s (thinking_mode=%s, drop_thinking=%s)", encoding_module_path,
                    thinking_mode, drop_thinking)

    @staticmethod
    def _adapt(messages):
        out = []
        for m in messages:
            m = dict(m)
            if "reasoning" in m and "reasoning_content" not in m:
                m["reasoning_content"] = m.pop("reasoning")
            out.append(m)
        return out

    def _keeps_thinking(self, messages) -> bool:
        # a conversation with tool definitions keeps every thinking block (the model needs them to follow the calls)
        return not self.drop_thinking or any(m.get("tools") for m in messages)

    def _prepare(self, messages):
        prepared = self._enc.merge_tool_messages(messages)
        prepared = self._enc.sort_tool_results_by_call_order(prepared)
        if not self._keeps_thinking(messages):
            prepared = self._enc._drop_thinking_messages(prepared)
        return prepared

    def _render(self, messages):
        drop = not self._keeps_thinking(messages)
        return [self._enc.render_message(i, messages, thinking_mode=self.thinking_mode, drop_thinking=drop,
                                         reasoning_effort=self.reasoning_effort if i == 0 else None)
                for i in range(len(messages))]

    def encode_messages_with_assistant_ranges(self, messages, tokenizer, eos_id):
        prepared = self._prepare(self._adapt(messages))
        rendered = self._render(prepared)
        text = "".join(rendered).rstrip("\n")
        tokens = tokenizer.encode(text, add_bos=True, add_eos=False)
        if not tokens or tokens[-1] != eos_id:
            tokens.append(eos_id)
        ranges: AssistantRanges = []
        prefix = ""
        for i, piece in enumerate(rendered):
            through = prefix + piece
            if prepared[i].get("role") == "assistant":
                a = tokenizer.encode(prefix, add_bos=True, add_eos=False)
                b = tokenizer.encode(through.rstrip("\n") if i == len(rendered) - 1 else through, add_bos=True,
                                     add_eos=False)
                if tokens[: len(a)] != a:
                    raise ValueError(f"DSV4 assistant span prefix alignment failed at message index {i}: prefix "
                                     "tokenization does not match full token prefix.")
                if tokens[: len(b)] != b:
                    raise ValueError(f"DSV4 assistant span boundary alignment failed at message index {i}: through "
                                     "tokenization does not match full token prefix.")
                end = len(b) + (1 if i == len(rendered) - 1 and len(tokens) == len(b) + 1 else 0)
                ranges.append((len(a), end))
            prefix = through
        return text, tokens, ranges


def build_chat_encoder(cfg) -> BaseChatEncoder | None:
    """From a `ChatEncoderConfig` / `DSV4EncoderConfig` (None → the tokenizer's template with the ChatML scan)."""
    if cfg is None:
        return None
    name = getattr(cfg, "name", "chatml")
    if name == "chatml":
        return ChatMLEncoder()
    if name == "dsv4":
        path = getattr(cfg, "encoding_path", "") or getattr(cfg, "encoding_module_path", "")
        return DSV4ChatEncoder(path, thinking_mode=getattr(cfg, "mode", "thinking"),
                               drop_thinking=getattr(cfg, "drop_thinking", True),
                               reasoning_effort=getattr(cfg, "reasoning_effort", None))
    raise ValueError(f"unknown chat encoder {name!r}")
