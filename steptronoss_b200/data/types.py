"""Types of the chat-JSON records (reference ``steptronoss/data/datasets/base_language_dataset.py``) and a checker
that says what is wrong with a record before a long templating job trips over it."""
from __future__ import annotations

from enum import Enum
from typing import Any, Literal, TypedDict


class Role(str, Enum):
    SYSTEM = "system"
    HUMAN = "human"
    USER = "user"
    ASSISTANT = "assistant"
    CONTEXT = "context"
    FUNCTION = "function"


class MessageContentType(str, Enum):
    TEXT = "text"
    CALL = "call"
    TOKEN = "token"


VALID_MESSAGE_CONTENT_TYPES = {m.value for m in MessageContentType}
VALID_ROLES = {r.value for r in Role}


class MessageContentPart(TypedDict, total=False):
    type: MessageContentType
    value: str
    loss_mask: Literal[0, 1] | None


class MessageItem(TypedDict, total=False):
    role: Role
    content: "str | list[MessageContentPart]"
    name: str | None
    loss_mask: Literal[0, 1]
    ground_truth: Any | None


class Dialog(TypedDict):
    conversations: list


def validate_dialog(record: dict) -> list:
    """Problems of one record as readable strings (empty list: the record is fine)."""
    problems = []
    conv = record.get("conversations") if isinstance(record, dict) else None
    if not isinstance(conv, list) or not conv:
        return ["'conversations' must be a non-empty list"]
    for i, turn in enumerate(conv):
        where = f"conversations[{i}]"
        if not isinstance(turn, dict):
            problems.append(f"{where} must be an object")
            continue
        if turn.get("role") not in VALID_ROLES:
            problems.append(f"{where}.role {turn.get('role')!r} is not one of {sorted(VALID_ROLES)}")
        content = turn.get("content")
        if isinstance(content, list):
            for j, part in enumerate(content):
                if not isinstance(part, dict) or part.get("type") not in VALID_MESSAGE_CONTENT_TYPES:
                    problems.append(f"{where}.content[{j}].type must be one of {sorted(VALID_MESSAGE_CONTENT_TYPES)}")
                elif not isinstance(part.get("value"), (str, list)):
                    problems.append(f"{where}.content[{j}].value must be text (or token ids)")
                if isinstance(part, dict) and part.get("loss_mask") not in (None, 0, 1):
                    problems.append(f"{where}.content[{j}].loss_mask must be 0, 1 or absent")
        elif not isinstance(content, str):
            problems.append(f"{where}.content must be text or a list of parts")
        if turn.get("loss_mask") not in (None, 0, 1):
            problems.append(f"{where}.loss_mask must be 0 or 1")
    if not any(isinstance(t, dict) and t.get("role") == Role.ASSISTANT.value for t in conv):
        problems.append("no assistant turn: nothing to train on")
    return problems
