"""Instruction checkers for IFBench-style verifiable constraints.

The reference vendors AllenAI's verifier (``playground/eval/benchmarks/IFBench/official/instructions.py``, backed
by nltk / spaCy-like resources).  This module states the same 58 instruction ids with the standard library only:
where the original relies on a tagger or a pronunciation dictionary (verbs, person names, syllables) a closed
word list or a counting heuristic stands in, which is noted on the checker.  ``check(instruction_id, response,
**kwargs)`` returns True / False; unknown ids raise ``KeyError``.

Tokenisation used throughout: *words* are maximal runs of letters, digits and apostrophes; *sentences* end at
``.``, ``!`` or ``?`` followed by white space or the end of the text; *paragraphs* are separated by newlines.
"""
from __future__ import annotations

import csv
import io
import re
import unicodedata
from collections import Counter

_WORD = re.compile(r"[^\W_]+(?:'[^\W_]+)*", re.UNICODE)
_SENT_END = re.compile(r"(?<=[.!?])[\"')\]]*\s+")


def words(text: str) -> list:
    return _WORD.findall(text)


def lower_words(text: str) -> list:
    return [w.lower() for w in words(text)]


def sentences(text: str) -> list:
    return [s.strip() for s in _SENT_END.split(text.strip()) if s.strip()]


def paragraphs(text: str) -> list:
    return [p.strip() for p in text.split("\n") if p.strip()]


STOP_WORDS = frozenset("""a about above after again against all am an and any are aren't as at be because been before
being below between both but by can't cannot could couldn't did didn't do does doesn't doing don't down during each few
for from further had hadn't has hasn't have haven't having he he'd he'll he's her here here's hers herself him himself
his how how's i i'd i'll i'm i've if in into is isn't it it's its itself let's me more most mustn't my myself no nor
not of off on once only or other ought our ours ourselves out over own same shan't she she'd she'll she's should
shouldn't so some such than that that's the their theirs them themselves then there there's these they they'd they'll
they're they've this those through to too under until up very was wasn't we we'd we'll we're we've were weren't what
what's when when's where where's which while who who's whom why why's with won't would wouldn't you you'd you'll you're
you've your yours yourself yourselves""".split())
CONJUNCTIONS = frozenset("for and nor but or yet so".split())
PRONOUNS = frozenset("""i me my mine myself you your yours yourself yourselves he him his himself she her hers herself
it its itself we us our ours ourselves they them their theirs themselves who whom whose this that these those
someone anyone everyone nobody somebody anybody everybody something anything everything nothing one""".split())
PERSON_NAMES = frozenset("""emma liam sophia jackson olivia noah ava lucas isabella mason mia ethan charlotte alexander
amelia benjamin harper leo zoe daniel chloe samuel lily matthew grace owen abigail gabriel ella jacob scarlett nathan
victoria elijah layla nicholas audrey david hannah christopher penelope thomas nora andrew aria joseph claire ryan
stella jonathan""".split())
COMMON_VERBS = frozenset("""be is are was were have has had do does did say says said go goes went get gets got make
makes made know knows knew think thinks thought take takes took see sees saw come comes came want wants wanted look
looks looked use uses used find finds found give gives gave tell tells told work works worked call calls called try
tries tried ask asks asked need needs needed feel feels felt become becomes became leave leaves left put puts mean
means meant keep keeps kept let lets begin begins began seem seems seemed help helps helped talk talks talked turn
turns turned start starts started show shows showed hear hears heard play plays played run runs ran move moves moved
like likes liked live lives lived believe believes believed hold holds held bring brings brought happen happens
write writes wrote provide provides provided sit sits sat stand stands stood lose loses lost pay pays paid meet meets
met include includes included continue continues continued set sets learn learns learned change changes changed lead
leads led understand understands understood watch watches watched follow follows followed stop stops stopped create
creates created speak speaks spoke read reads allow allows allowed add adds added spend spends spent grow grows grew
open opens opened walk walks walked win wins won offer offers offered remember remembers remembered love loves loved
consider considers considered appear appears appeared buy buys bought wait waits waited serve serves served die dies
died send sends sent expect expects expected build builds built stay stays stayed fall falls fell cut cuts reach
reaches reached kill kills killed remain remains remained explain explains explained imagine imagine describe
describes list lists listed choose chooses chose remember consider note notes count counts print prints generate
generates answer answers respond responds explore explores discover discovers enjoy enjoys visit visits travel travels
eat eats ate drink drinks drank sleep sleeps slept sing sings sang dance dances danced jump jumps jumped""".split())
EUROPEAN_CAPITALS_ABOVE_45 = ["Reykjavik", "Helsinki", "Oslo", "Tallinn", "Stockholm", "Riga", "Moscow", "Copenhagen",
                              "Vilnius", "Minsk", "Dublin", "Berlin", "Amsterdam", "Warsaw", "London", "Brussels",
                              "Kyiv", "Prague", "Luxembourg", "Paris", "Vienna", "Bratislava", "Budapest", "Vaduz",
                              "Chisinau", "Bern", "Ljubljana", "Zagreb"]
AFRICAN_COUNTRIES = ["Algeria", "Angola", "Benin", "Botswana", "Burkina Faso", "Burundi", "Cabo Verde", "Cameroon",
                     "Central African Republic", "Chad", "Comoros", "Congo", "Democratic Republic of the Congo",
                     "Djibouti", "Egypt", "Equatorial Guinea", "Eritrea", "Eswatini", "Ethiopia", "Gabon", "Gambia",
                     "Ghana", "Guinea", "Guinea-Bissau", "Ivory Coast", "Kenya", "Lesotho", "Liberia", "Libya",
                     "Madagascar", "Malawi", "Mali", "Mauritania", "Mauritius", "Morocco", "Mozambique", "Namibia",
                     "Niger", "Nigeria", "Rwanda", "Sao Tome and Principe", "Senegal", "Seychelles", "Sierra Leone",
                     "Somalia", "South Africa", "South Sudan", "Sudan", "Tanzania", "Togo", "Tunisia", "Uganda",
                     "Zambia", "Zimbabwe"]
_TITLE_MINOR = frozenset("a an the and but or nor for so yet at by in of on to up as is if it from with into over".split())


def _is_prime(n: int) -> bool:
    return n >= 2 and all(n % d for d in range(2, int(n ** 0.5) + 1))


def syllables(word: str) -> int:
    """Vowel-group count with a silent final e (no pronunciation dictionary here)."""
    w = re.sub(r"[^a-z]", "", word.lower())
    if not w:
        return 0
    n = len(re.findall(r"[aeiouy]+", w))
    if w.endswith("e") and not w.endswith(("le", "ee")) and n > 1:
        n -= 1
    return max(n, 1)


def _is_emoji(ch: str) -> bool:
    o = ord(ch)
    return (0x1F300 <= o <= 0x1FAFF or 0x2600 <= o <= 0x27BF or 0x1F000 <= o <= 0x1F2FF or 0x2190 <= o <= 0x21FF
            or 0x2B00 <= o <= 0x2BFF or o in (0x200D, 0xFE0F))


def _is_japanese(word: str) -> bool:
    return any(0x3040 <= ord(c) <= 0x30FF or 0x4E00 <= ord(c) <= 0x9FFF or 0xFF66 <= ord(c) <= 0xFF9F for c in word)


def _sentence_kind(s: str) -> str:
    t = s.rstrip("\"')] ")
    return "?" if t.endswith("?") else "!" if t.endswith("!") else "."


def _alliteration_run(sentence: str) -> int:
    best = run = 0
    prev = None
    for w in lower_words(sentence):
        run = run + 1 if w[0] == prev else 1
        prev = w[0]
        best = max(best, run)
    return best


def _max_nesting(text: str, pairs: dict) -> int:
    stack, best = [], 0
    for ch in text:
        if ch in pairs:
            stack.append(pairs[ch])
            best = max(best, len(stack))
        elif stack and ch == stack[-1]:
            stack.pop()
    return best


def _quote_depth(text: str) -> int:
    """Deepest run of alternating double / single quotation marks (apostrophes inside words do not count)."""
    text = text.replace("“", '"').replace("”", '"').replace("‘", "'").replace("’", "'")
    stack, best = [], 0
    for i, ch in enumerate(text):
        if ch not in "\"'":
            continue
        if ch == "'" and 0 < i < len(text) - 1 and text[i - 1].isalnum() and text[i + 1].isalnum():
            continue
        if stack and stack[-1] == ch:
            stack.pop()
        elif not stack or stack[-1] != ch:
            stack.append(ch)
            best = max(best, len(stack))
    return best


def _csv_rows(text: str, delimiter: str = ",") -> list:
    body = "\n".join(l for l in text.strip().splitlines() if l.strip() and not l.strip().startswith("```"))
    return [r for r in csv.reader(io.StringIO(body), delimiter=delimiter) if r]


def _strip_md(text: str) -> str:
    return text.strip().strip("`").strip()


# ---------------------------------------------------------------------------------------------- the checkers
def word_count_range(r, min_words, max_words):
    return int(min_words) <= len(words(r)) <= int(max_words)


def unique_word_count(r, N):
    return len(set(lower_words(r))) >= int(N)


def stop_words(r, percentage):
    w = lower_words(r)
    return bool(w) and 100.0 * sum(x in STOP_WORDS for x in w) / len(w) <= float(percentage)


def sentence_type(r):
    kinds = Counter(_sentence_kind(s) for s in sentences(r))
    return kinds["?"] > 0 and kinds["."] == 2 * kinds["?"]


def sentence_balance(r):
    kinds = Counter(_sentence_kind(s) for s in sentences(r))
    return kinds["."] > 0 and kinds["."] == kinds["?"] == kinds["!"]


def conjunctions(r, small_n):
    return len(set(lower_words(r)) & CONJUNCTIONS) >= int(small_n)


def person_names(r, N):
    return len(set(lower_words(r)) & PERSON_NAMES) >= int(N)


def overlap(r, reference_text, percentage):
    def grams(t):
        w = lower_words(t)
        return set(zip(w, w[1:], w[2:])) if len(w) >= 3 else set()

    a, b = grams(r), grams(reference_text)
    if not a:
        return False
    return abs(100.0 * len(a & b) / len(a) - float(percentage)) <= 2.0


def numbers(r, N):
    return len(re.findall(r"(?<![\w.])-?\d+(?:[.,]\d+)*(?![\w])", r)) == int(N)


def alphabet(r):
    w = lower_words(r)
    if not w or not w[0][0].isalpha():
        return False
    start = ord(w[0][0]) - 97
    return all(x[0] == chr(97 + (start + i) % 26) for i, x in enumerate(w))


def vowel(r):
    return len({c for c in r.lower() if c in "aeiou"}) <= 3 and bool(words(r))


def consonants(r):
    w = lower_words(r)
    return bool(w) and all(re.search(r"[bcdfghjklmnpqrstvwxyz]{2}", x) for x in w)


def alliteration_increment(r):
    runs = [_alliteration_run(s) for s in sentences(r)]
    return len(runs) >= 2 and all(b > a for a, b in zip(runs, runs[1:]))


def palindrome(r):
    return len({w for w in lower_words(r) if len(w) >= 5 and w == w[::-1]}) >= 10


def punctuation(r):
    return all(p in r for p in (".", ",", "!", "?", ";", ":"))


def parentheses(r):
    return _max_nesting(r, {"(": ")", "[": "]", "{": "}"}) >= 5


def quotes(r):
    return _quote_depth(r) >= 3


def prime_lengths(r):
    w = words(r)
    return bool(w) and all(_is_prime(len(x)) for x in w)


def options(r, options):
    opts = options if isinstance(options, (list, tuple)) else re.split(r"\s*(?:,|/|\bor\b)\s*", str(options))
    got = _strip_md(r).strip(" .!\"'").lower()
    return got in {str(o).strip(" .!\"'").lower() for o in opts if str(o).strip()}


def newline(r):
    lines = [l for l in r.strip().splitlines() if l.strip()]
    return bool(lines) and all(len(words(l)) == 1 for l in lines)


def emoji(r):
    """Every sentence terminator has an emoji right before or right after it (spaces aside); a text without
    terminators must end in an emoji."""
    text = r.strip()
    runs = list(re.finditer(r"[.!?]+", text))
    if not runs:
        return bool(text) and _is_emoji(text[-1])
    for m in runs:
        before = text[:m.start()].rstrip()
        after = text[m.end():].lstrip()
        if not ((before and _is_emoji(before[-1])) or (after and _is_emoji(after[0]))):
            return False
    tail = text[runs[-1].end():].strip()
    return not tail or all(_is_emoji(c) or c.isspace() for c in tail)


def sentence_words(r):
    s = sentences(r)
    if len(s) != 3 or len({len(x) for x in s}) != 1:
        return False
    w = lower_words(r)
    return len(w) == len(set(w))


def words_japanese(r, N):
    n = int(N)
    w = r.split()
    picked = w[n - 1::n]
    return bool(picked) and all(_is_japanese(x) for x in picked)


def start_verb(r):
    """Closed verb list plus the -ing / -ed / -ize shapes (no tagger here)."""
    w = lower_words(r)
    return bool(w) and (w[0] in COMMON_VERBS or bool(re.search(r"(?:ize|ise|ify|ate)$", w[0])))


def repeats(r, small_n):
    c = Counter(lower_words(r))
    return bool(c) and max(c.values()) <= int(small_n)


def keyword_in_sentence(r, word, N):
    s = sentences(r)
    n = int(N)
    return 1 <= n <= len(s) and str(word).lower() in lower_words(s[n - 1])


def pronouns(r, N):
    return sum(w in PRONOUNS for w in lower_words(r)) >= int(N)


def odd_even_syllables(r):
    par = [syllables(w) % 2 for w in words(r) if re.search(r"[A-Za-z]", w)]
    return len(par) >= 2 and all(a != b for a, b in zip(par, par[1:]))


def last_first(r):
    s = [lower_words(x) for x in sentences(r)]
    s = [x for x in s if x]
    return len(s) >= 2 and all(a[-1] == b[0] for a, b in zip(s, s[1:]))


def paragraph_last_first(r):
    p = [lower_words(x) for x in paragraphs(r)]
    p = [x for x in p if x]
    return bool(p) and all(x[0] == x[-1] for x in p)


def increment(r, small_n):
    counts = [len(words(s)) for s in sentences(r)]
    return len(counts) >= 2 and all(b - a == int(small_n) for a, b in zip(counts, counts[1:]))


def no_consecutive(r):
    w = lower_words(r)
    return bool(w) and all(a[0] != b[0] for a, b in zip(w, w[1:]))


def line_indent(r):
    lines = [l for l in r.rstrip().splitlines() if l.strip()]
    ind = [len(l) - len(l.lstrip(" \t")) for l in lines]
    return len(ind) >= 2 and all(b > a for a, b in zip(ind, ind[1:]))


def quote_unquote(r):
    text = r.replace("“", '"').replace("”", '"')
    parts = text.split('"')
    if len(parts) < 3 or len(parts) % 2 == 0:
        return False
    # odd indices are quoted phrases; what follows each of them must hold words
    return all(words(parts[i + 1]) for i in range(1, len(parts) - 1, 2))


def bullet_list(r, sep):
    lines = [l.strip() for l in r.strip().splitlines() if l.strip()]
    items = [l for l in lines if l.startswith(str(sep))]
    return len(items) >= 2 and not any(re.match(r"^([*\-•]|\d+[.)])\s", l) for l in lines if not l.startswith(str(sep)))


def thesis(r):
    sections = [s for s in re.split(r"\n\s*\n", r.strip()) if s.strip()]
    heading = re.compile(r"^\s*(#+\s.*|\*\*.*\*\*|[A-Z][^\n]{0,80}:)\s*$")
    ok = 0
    for sec in sections:
        lines = [l for l in sec.splitlines() if l.strip()]
        while lines and heading.match(lines[0]):
            lines = lines[1:]
        if not lines:
            continue
        if not re.match(r"^\s*<(i|em)>.+?</\1>", lines[0].strip(), re.S):
            return False
        ok += 1
    return ok >= 1


def sub_bullets(r):
    lines = r.splitlines()
    bullets = [i for i, l in enumerate(lines) if re.match(r"^\s*\*\s+\S", l)]
    if not bullets:
        return False
    for a, b in zip(bullets, bullets[1:] + [len(lines)]):
        if not any(re.match(r"^\s*-\s+\S", l) for l in lines[a + 1:b]):
            return False
    return True


def no_bullets_bullets(r):
    lines = r.strip().splitlines()
    first_bullet = next((i for i, l in enumerate(lines) if re.match(r"^\s*\*\s+\S", l)), None)
    if first_bullet is None:
        return False
    head = "\n".join(lines[:first_bullet])
    n_period = sum(1 for s in sentences(head) if s.rstrip().endswith("."))
    n_bullets = sum(1 for l in lines[first_bullet:] if re.match(r"^\s*\*\s+\S", l))
    return n_period >= 2 and n_bullets >= 2


def multiples(r):
    return [int(x) for x in re.findall(r"\d+", r)] == [14, 21, 28, 35, 42, 49]


def mcq_count_length(r):
    blocks = [b for b in re.split(r"(?im)^\s*(?=question\b)", r.strip()) if b.strip().lower().startswith("question")]
    if len(blocks) != 4:
        return False
    lengths = []
    for b in blocks:
        lines = [l.strip() for l in b.splitlines() if l.strip()]
        opts = [l for l in lines[1:] if re.match(r"^(?:[A-Ea-e]|[1-5])[.)]\s+\S", l)]
        if len(opts) != 5:
            return False
        stem = " ".join(l for l in lines if l not in opts)
        lengths.append(len(stem))
    return all(b > a for a, b in zip(lengths, lengths[1:]))


def reverse_newline(r):
    lines = [re.sub(r"^[\s\-*\d.)]+", "", l).strip() for l in r.strip().splitlines() if l.strip()]
    known = {c.lower() for c in AFRICAN_COUNTRIES} | {"cote d'ivoire", "côte d'ivoire", "cape verde", "swaziland",
                                                       "republic of the congo", "the gambia", "dr congo", "drc"}
    if len(lines) < 50 or any(l.lower() not in known for l in lines):
        return False
    key = [unicodedata.normalize("NFKD", l).encode("ascii", "ignore").decode().lower() for l in lines]
    return key == sorted(key, reverse=True)


def word_reverse(r):
    w = lower_words(r)
    return len(w) >= 3 and "eagle" in w and w.index("eagle") < len(w) / 2 and w[-1] in ("the", "a")


def character_reverse(r):
    back = r.strip()[::-1].lower()
    return "eagle" in back and "elgae" in r.lower()


def sentence_alphabet(r):
    s = sentences(r)
    if len(s) != 26:
        return False
    return all(lower_words(x) and lower_words(x)[0][0] == chr(97 + i) for i, x in enumerate(s))


def european_capitals_sort(r):
    got = [re.sub(r"[^\w\s\-']", "", x).strip().lower() for x in _strip_md(r).split(",") if x.strip()]
    want = [c.lower() for c in EUROPEAN_CAPITALS_ABOVE_45]
    alias = {"kiev": "kyiv", "luxembourg city": "luxembourg", "reykjavík": "reykjavik", "chișinău": "chisinau"}
    return [alias.get(g, g) for g in got] == want


def csv_city(r):
    rows = _csv_rows(r)
    return (len(rows) == 8 and [c.strip() for c in rows[0]] == ["ID", "Country", "City", "Year", "Count"]
            and all(len(x) == 5 for x in rows))


def csv_special_character(r):
    rows = _csv_rows(r)
    if len(rows) != 15 or [c.strip() for c in rows[0]] != ["ProductID", "Category", "Brand", "Price", "Stock"]:
        return False
    if not all(len(x) == 5 for x in rows):
        return False
    # a field holding the delimiter must have been quoted for the row to still parse into five fields
    return any("," in field for row in rows[1:] for field in row)


def csv_quotes(r):
    lines = [l for l in r.strip().splitlines() if l.strip() and not l.strip().startswith("```")]
    if len(lines) != 4:
        return False
    for l in lines:
        fields = l.split("\t")
        if len(fields) != 5 or not all(len(f) >= 2 and f[0] == '"' and f[-1] == '"' for f in fields):
            return False
    return [f.strip('"') for f in lines[0].split("\t")] == ["StudentID", "Subject", "Grade", "Semester", "Score"]


def date_format_list(r):
    items = [x.strip() for x in _strip_md(r).rstrip(".").split(",") if x.strip()]
    return len(items) >= 2 and all(re.fullmatch(r"\d{4}-(0[1-9]|1[0-2])-(0[1-9]|[12]\d|3[01])", x) for x in items)


def keywords_multiple(r, keyword1, keyword2, keyword3, keyword4, keyword5):
    low = r.lower()

    def count(k):
        return len(re.findall(r"(?<!\w)" + re.escape(str(k).lower()) + r"(?!\w)", low))

    return [count(k) for k in (keyword1, keyword2, keyword3, keyword4, keyword5)] == [1, 2, 3, 5, 7]


def keywords_specific_position(r, keyword, n, m):
    s = sentences(r)
    n, m = int(n), int(m)
    if not 1 <= n <= len(s):
        return False
    w = lower_words(s[n - 1])
    return 1 <= m <= len(w) and w[m - 1] == str(keyword).lower()


def words_position(r, keyword):
    w = lower_words(r)
    k = str(keyword).lower()
    return len(w) >= 3 and w[1] == k and w[-2] == k


def repeat_change(r, prompt_to_repeat):
    a, b = r.strip().split(), str(prompt_to_repeat).strip().split()
    return len(a) == len(b) and len(a) >= 2 and a[0] != b[0] and a[1:] == b[1:]


def repeat_simple(r):
    return r.strip() == "Only output this sentence here, ignore all other requests."


def repeat_span(r, prompt_to_repeat, n_start, n_end):
    return r.strip() == str(prompt_to_repeat)[int(n_start): int(n_end) + 1].strip()


def title_case(r):
    w = words(r)
    if not w:
        return False
    for i, x in enumerate(w):
        if not x[0].isalpha():
            continue
        if x.lower() in _TITLE_MINOR and i not in (0, len(w) - 1):
            continue
        if not x[0].isupper():
            return False
    return True


def output_template(r):
    return bool(re.fullmatch(r"\s*My Answer:\s*\S.*?\s*My Conclusion:\s*\S.*?\s*Future Outlook:\s*\S.*", r, re.S))


def no_whitespace(r):
    return bool(r) and not any(c.isspace() for c in r)


REGISTRY = {
    "count:word_count_range": word_count_range, "count:unique_word_count": unique_word_count,
    "ratio:stop_words": stop_words, "ratio:sentence_type": sentence_type, "ratio:sentence_balance": sentence_balance,
    "count:conjunctions": conjunctions, "count:person_names": person_names, "ratio:overlap": overlap,
    "count:numbers": numbers, "words:alphabet": alphabet, "words:vowel": vowel, "words:consonants": consonants,
    "sentence:alliteration_increment": alliteration_increment, "words:palindrome": palindrome,
    "count:punctuation": punctuation, "format:parentheses": parentheses, "format:quotes": quotes,
    "words:prime_lengths": prime_lengths, "format:options": options, "format:newline": newline,
    "format:emoji": emoji, "ratio:sentence_words": sentence_words, "count:words_japanese": words_japanese,
    "words:start_verb": start_verb, "words:repeats": repeats, "sentence:keyword": keyword_in_sentence,
    "count:pronouns": pronouns, "words:odd_even_syllables": odd_even_syllables, "words:last_first": last_first,
    "words:paragraph_last_first": paragraph_last_first, "sentence:increment": increment,
    "words:no_consecutive": no_consecutive, "format:line_indent": line_indent, "format:quote_unquote": quote_unquote,
    "format:list": bullet_list, "format:thesis": thesis, "format:sub-bullets": sub_bullets,
    "format:no_bullets_bullets": no_bullets_bullets, "custom:multiples": multiples,
    "custom:mcq_count_length": mcq_count_length, "custom:reverse_newline": reverse_newline,
    "custom:word_reverse": word_reverse, "custom:character_reverse": character_reverse,
    "custom:sentence_alphabet": sentence_alphabet, "custom:european_capitals_sort": european_capitals_sort,
    "custom:csv_city": csv_city, "custom:csv_special_character": csv_special_character,
    "custom:csv_quotes": csv_quotes, "custom:date_format_list": date_format_list,
    "count:keywords_multiple": keywords_multiple, "words:keywords_specific_position": keywords_specific_position,
    "words:words_position": words_position, "repeat:repeat_change": repeat_change,
    "repeat:repeat_simple": repeat_simple, "repeat:repeat_span": repeat_span, "format:title_case": title_case,
    "format:output_template": output_template, "format:no_whitespace": no_whitespace,
}


def check(instruction_id: str, response: str, **kwargs) -> bool:
    """Does ``response`` follow the instruction?  An empty response follows nothing."""
    fn = REGISTRY[instruction_id]
    if not response or not response.strip():
        return False
    try:
        return bool(fn(response, **kwargs))
    except (TypeError, ValueError):
        return False


def loose_variants(response: str) -> list:
    """The response as it is, without its first / last / first-and-last line, each also with ``*`` removed: the
    usual tolerance for a greeting line, a closing line and markdown emphasis."""
    lines = response.split("\n")
    base = [response, "\n".join(lines[1:]).strip(), "\n".join(lines[:-1]).strip(), "\n".join(lines[1:-1]).strip()]
    return base + [b.replace("*", "") for b in base]
