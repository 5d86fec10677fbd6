import pytest

from steptronoss_b200.text_processing import content_parsing as cp
from steptronoss_b200.text_processing import math_utils as mu


def _brute(s):
    n = len(s)
    suf = sorted(range(n), key=lambda i: s[i:])
    tot = 0
    for a, b in zip(suf, suf[1:]):
        k = 0
        while a + k < n and b + k < n and s[a + k] == s[b + k]:
            k += 1
        tot += k
    return tot * 2 / (n * (n + 1))


@pytest.mark.parametrize("s", ["abcdefg", "aaaaaaaa", "abababababab", "the cat sat on the mat, the cat sat", "日本語日本語"])
def test_repeatness_matches_brute_force(s):
    assert abs(mu.repeatness_score(s) - _brute(s)) < 1e-12


def test_repeatness_flags_loops():
    assert mu.repeatness("wait, let me think. " * 30) and not mu.repeatness("A short distinct sentence about kernels.")


def test_boxed_extraction_and_equality():
    sol = r"so we get \boxed{1} and finally \boxed{\frac{3}{4}}."
    assert mu.last_boxed_only_string(sol) == r"\boxed{\frac{3}{4}}"
    assert mu.get_answer_str(sol) == r"\frac{3}{4}"
    assert mu.get_final_answer("The answer is: 42.") == "42"
    assert mu.is_equiv(r"\dfrac{3}{4}", "3/4") and mu.is_equiv("0.5", r"\frac12") and mu.is_equiv("x = 7", "7")
    assert not mu.is_equiv("3", "4")
    assert mu.normalize_final_answer("100,000 dollars") == "100000"
    assert mu.normalize_final_answer(r"$\frac12$") == r"\frac{1}{2}"


def test_think_and_solution_parsing():
    r = "<think>first\nsecond</think>\nThe answer is 4<|im_end|>tail"
    assert cp.parse_reason_reasoning_content(r) == "first\nsecond"
    assert cp.parse_reason_solution(r) == "The answer is 4"
    assert cp.parse_reason_solution("<think>never closes") == ""
    assert cp.parse_chat_solution("hello<|im_end|>x") == "hello" and cp.parse_chat_solution("hello") == ""
