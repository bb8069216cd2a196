"""Core public types (parity: reference ``src/art/types.py:1-19``)."""
from __future__ import annotations

from typing import Literal

import pydantic
from openai.types.chat.chat_completion import Choice
from openai.types.chat.chat_completion_message_param import ChatCompletionMessageParam
from openai.types.chat.chat_completion_tool_param import ChatCompletionToolParam

Message = ChatCompletionMessageParam
MessageOrChoice = Message | Choice
Messages = list[Message]
MessagesAndChoices = list[MessageOrChoice]
Tools = list[ChatCompletionToolParam]
Verbosity = Literal[0, 1, 2]


class TrainConfig(pydantic.BaseModel):
    """Public per-call training knobs: AdamW learning rate and the KL weight ``beta``."""

    learning_rate: float = 5e-6
    beta: float = 0.0
