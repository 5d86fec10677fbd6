"""Split a model response into its reasoning and its solution (reference
``steptronoss/text_processing/content_parsing.py:1-39``)."""
IM_END_TOKEN = "<|im_end|>"
THINK_BEGIN_TOKEN = "<think>"
THINK_END_TOKEN = "</think>"
THINK_END_WITH_NEWLINE = THINK_END_TOKEN + "\n"


def parse_chat_reasoning_content(response: str) -> str:
    """A plain chat response carries no reasoning block."""
    return ""


def parse_chat_solution(response: str) -> str:
    """Text before the first end-of-message token; empty when the response was cut before it."""
    head, sep, _ = response.partition(IM_END_TOKEN)
    return head if sep else ""


def parse_reason_reasoning_content(response: str) -> str:
    """Everything up to the last ``</think>`` (minus the opening tag); the whole text if it never closes."""
    body, sep, _ = response.rpartition(THINK_END_TOKEN)
    if not sep:
        return response.strip("\n")
    body = body.replace(THINK_END_TOKEN, "")
    first, opened, rest = body.partition(THINK_BEGIN_TOKEN)
    if opened:
        body = rest.replace(THINK_BEGIN_TOKEN, "")
    return body.strip("\n")


def parse_reason_solution(response: str) -> str:
    """Text between the last ``</think>\\n`` and the end-of-message token; empty if either is missing."""
    _, sep, tail = response.rpartition(THINK_END_WITH_NEWLINE)
    if not sep:
        return ""
    head, end, _ = tail.partition(IM_END_TOKEN)
    return head if end else ""
