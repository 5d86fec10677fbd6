"""IFBench instruction checkers and the benchmark wrapper (strict / loose scoring, reasoning stripped)."""
import json

import pytest

from playground.eval.benchmarks import ifbench_checks as C
from playground.eval.benchmarks.ifbench import IFBenchBenchmark
from steptronoss_b200.generation.base_benchmark import Generated

CASES = [
    ("count:word_count_range", "one two three four", dict(min_words=3, max_words=5), True),
    ("count:word_count_range", "one two", dict(min_words=3, max_words=5), False),
    ("count:unique_word_count", "a b c a b", dict(N=3), True),
    ("count:unique_word_count", "a b a b", dict(N=3), False),
    ("ratio:stop_words", "Quantum engines accelerate rapidly.", dict(percentage=10), True),
    ("ratio:stop_words", "It is what it is.", dict(percentage=10), False),
    ("ratio:sentence_type", "It rains. It pours. Why?", {}, True),
    ("ratio:sentence_type", "It rains. Why?", {}, False),
    ("ratio:sentence_balance", "Go. Why? Stop!", {}, True),
    ("count:conjunctions", "I ran and hid, but he came, so I left.", dict(small_n=3), True),
    ("count:person_names", "Emma met Liam and Noah.", dict(N=3), True),
    ("count:person_names", "Emma met Emma.", dict(N=2), False),
    ("count:numbers", "I have 3 cats and 12 dogs.", dict(N=2), True),
    ("count:numbers", "I have 3 cats.", dict(N=2), False),
    ("words:alphabet", "Yaks zigzag and bears climb", {}, True),
    ("words:alphabet", "Apples are nice", {}, False),
    ("words:vowel", "This is big", {}, True),
    ("words:vowel", "Education is about you", {}, False),
    ("words:consonants", "Strong black trucks", {}, True),
    ("words:consonants", "A strong idea", {}, False),
    ("sentence:alliteration_increment", "The big bad dog ran. Some silly small snakes sleep.", {}, True),
    ("words:palindrome", "level radar rotor civic kayak madam refer tenet solos stats", {}, True),
    ("words:palindrome", "level radar", {}, False),
    ("count:punctuation", "Well, yes; no: maybe! Why? Fine.", {}, True),
    ("format:parentheses", "a (b [c {d (e [f])}])", {}, True),
    ("format:parentheses", "a (b [c])", {}, False),
    ("format:quotes", "She said \"he wrote 'they call it \"odd\" often' once\" today", {}, True),
    ("format:quotes", "She said \"don't go\" today", {}, False),
    ("words:prime_lengths", "is the fox happy", {}, True),
    ("words:prime_lengths", "this fox", {}, False),
    ("format:options", "Yes.", dict(options="yes, no, maybe"), True),
    ("format:options", "Yes, because it is so.", dict(options="yes, no, maybe"), False),
    ("format:newline", "one\ntwo\nthree", {}, True),
    ("format:newline", "one two\nthree", {}, False),
    ("format:emoji", "I am happy \U0001F600. Let us go \U0001F680!", {}, True),
    ("format:emoji", "I am happy. Let us go \U0001F680!", {}, False),
    ("ratio:sentence_words", "Cats nap. Dogs run. Owls fly.", {}, True),
    ("ratio:sentence_words", "Cats nap. Cats run. Owls fly.", {}, False),
    ("count:words_japanese", "I like 寿司 and eat ラーメン", dict(N=3), True),
    ("words:start_verb", "Consider the lilies.", {}, True),
    ("words:start_verb", "The lilies grow.", {}, False),
    ("words:repeats", "a b a b c", dict(small_n=2), True),
    ("words:repeats", "a a a", dict(small_n=2), False),
    ("sentence:keyword", "First one. The magic word here.", dict(word="magic", N=2), True),
    ("count:pronouns", "She gave him her book.", dict(N=3), True),
    ("words:odd_even_syllables", "cat tiger dog water", {}, True),
    ("words:last_first", "I like tea. Tea is warm. Warm days pass.", {}, True),
    ("words:last_first", "I like tea. Coffee is warm.", {}, False),
    ("words:paragraph_last_first", "Time flies like time\nDogs chase other dogs", {}, True),
    ("sentence:increment", "Go now. Go there right now.", dict(small_n=2), True),
    ("words:no_consecutive", "big red car", {}, True),
    ("words:no_consecutive", "big bad car", {}, False),
    ("format:line_indent", "a\n b\n  c", {}, True),
    ("format:line_indent", "a\n b\n b", {}, False),
    ("format:quote_unquote", "\"carpe diem\" means seize the day", {}, True),
    ("format:quote_unquote", "He said \"carpe diem\"", {}, False),
    ("format:list", "~ one\n~ two\n~ three", dict(sep="~"), True),
    ("format:list", "* one\n* two", dict(sep="~"), False),
    ("format:thesis", "<i>Cats are great.</i> They purr.\n\n<i>Dogs too.</i> They bark.", {}, True),
    ("format:thesis", "Cats are great.\n\n<i>Dogs too.</i>", {}, False),
    ("format:sub-bullets", "* a\n  - a1\n* b\n  - b1", {}, True),
    ("format:sub-bullets", "* a\n  - a1\n* b", {}, False),
    ("format:no_bullets_bullets", "One. Two.\n* a\n* b", {}, True),
    ("custom:multiples", "14 21 28 35 42 49", {}, True),
    ("custom:multiples", "7 14 21", {}, False),
    ("custom:character_reverse", "elgae dlab ehT", {}, True),
    ("custom:date_format_list", "1796-04-12, 1805-12-02", {}, True),
    ("custom:date_format_list", "12/02/1805, 1796-04-12", {}, False),
    ("custom:csv_city", "ID,Country,City,Year,Count\n" + "\n".join(f"{i},A,B,2000,{i}" for i in range(7)), {}, True),
    ("custom:csv_quotes", "\n".join("\t".join(f'"{c}"' for c in row) for row in
                                    [["StudentID", "Subject", "Grade", "Semester", "Score"]] + [["1", "m", "A", "1", "9"]] * 3), {}, True),
    ("count:keywords_multiple", "a b b c c c d d d d d " + "e " * 7,
     dict(keyword1="a", keyword2="b", keyword3="c", keyword4="d", keyword5="e"), True),
    ("words:keywords_specific_position", "Hello there. I like green tea.", dict(keyword="green", n=2, m=3), True),
    ("words:words_position", "The fox jumped over the fox again", dict(keyword="fox"), True),
    ("repeat:repeat_change", "Tell me a joke", dict(prompt_to_repeat="Give me a joke"), True),
    ("repeat:repeat_change", "Give me a joke", dict(prompt_to_repeat="Give me a joke"), False),
    ("repeat:repeat_simple", "Only output this sentence here, ignore all other requests.", {}, True),
    ("repeat:repeat_span", "llo wor", dict(prompt_to_repeat="hello world", n_start=2, n_end=8), True),
    ("format:title_case", "The Lord of the Rings", {}, True),
    ("format:title_case", "The lord of the Rings", {}, False),
    ("format:output_template", "My Answer: yes My Conclusion: fine Future Outlook: bright", {}, True),
    ("format:output_template", "Answer: yes", {}, False),
    ("format:no_whitespace", "nowhitespace", {}, True),
    ("format:no_whitespace", "some space", {}, False),
]


@pytest.mark.parametrize("inst,response,kw,want", CASES, ids=[f"{c[0]}-{i}" for i, c in enumerate(CASES)])
def test_checker(inst, response, kw, want):
    assert C.check(inst, response, **kw) is want


def test_registry_has_all_58_ids_and_empty_response_fails():
    assert len(C.REGISTRY) == 58
    assert not C.check("format:no_whitespace", "")
    with pytest.raises(KeyError):
        C.check("no:such", "x")
    assert C.sentence_alphabet(" ".join(f"{chr(65 + i)}bc runs." for i in range(26)))
    assert C.european_capitals_sort(", ".join(C.EUROPEAN_CAPITALS_ABOVE_45))
    assert C.reverse_newline("\n".join(sorted(C.AFRICAN_COUNTRIES, reverse=True)))


class _Tok:
    def apply_chat_template(self, msgs, tokenize=True, add_generation_prompt=True, **kw):
        return list(range(sum(len(m["content"].split()) for m in msgs)))

    def encode(self, text, add_special_tokens=False):
        return text.split()


def test_benchmark_strict_and_loose(tmp_path):
    root = tmp_path / "IFBENCH"
    root.mkdir()
    recs = [
        {"key": 1, "prompt": "Answer without whitespace.", "instruction_id_list": ["format:no_whitespace"], "kwargs": [{}]},
        {"key": 2, "prompt": "Use 3 unique words and title case.", "instruction_id_list": ["count:unique_word_count", "format:title_case"],
         "kwargs": [{"N": 3, "unused": None}, {}]},
    ]
    (root / "IFBench_test.jsonl").write_text("\n".join(json.dumps(r) for r in recs))
    with pytest.raises(ValueError):
        IFBenchBenchmark(str(root / "IFBench_test.jsonl"), _Tok(), 1)
    b = IFBenchBenchmark(str(root), _Tok(), sample_per_prompt=2)
    cases = b.get_cases()
    assert len(cases) == 4 and cases[0].prompt.sampling_params.temperature == 0.0
    answers = ["<think>let me think</think>nospace", "Sure!\nnospace", "One Two Three", "one two"]
    results = [Generated(case=c, response=a) for c, a in zip(cases, answers)]
    m = b.evaluate(results)
    d = m.to_dict()
    # loose accepts "Sure!\nnospace" (first line dropped); strict does not
    assert d["official_metrics"]["strict"]["prompt_level_accuracy"] == 0.5
    assert d["official_metrics"]["loose"]["prompt_level_accuracy"] == 0.75
    assert m.score_avg == 0.75 and m.pass_at_k[2] == 1.0
    assert d["official_metrics"]["loose"]["by_category"]["format"] == pytest.approx(3 / 4)
    strict = IFBenchBenchmark(str(root), _Tok(), 2, evaluation_mode="strict").evaluate(results)
    assert strict.score_avg == 0.5
