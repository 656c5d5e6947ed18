"""Ten small MBPP-style problems bundled for smoke tests of code generation (plain equality checks, no special oracles).

Schema per task (same as the reference's evals/mbpp_lite.py:4-150 and the MBPP+ release): ``entry_point``, ``prompt``
(signature + docstring), ``canonical_solution`` (body that completes the prompt), ``base_input`` / ``plus_input`` (lists of
argument lists) and ``atol``.  Ids live in the ``Mbpp/100xx`` range, which the real dataset does not use.
"""


def _task(entry, signature, doc, body, base, plus, atol=0.0):
    prompt = f'def {signature}:\n    """{doc}\n    """\n'
    return {"entry_point": entry, "prompt": prompt, "canonical_solution": body, "base_input": base, "plus_input": plus, "atol": atol}


DATA = {
    "Mbpp/10001": _task(
        "count_vowels", "count_vowels(s: str) -> int", "Return how many characters of s are vowels (aeiou, either case).",
        "    return sum(ch in 'aeiouAEIOU' for ch in s)\n",
        [["banana"], ["sky"], [""]], [["AEIOU"], ["Programming"], ["xyz"]]),
    "Mbpp/10002": _task(
        "gcd", "gcd(a: int, b: int) -> int", "Greatest common divisor of two non-negative integers.",
        "    while b:\n        a, b = b, a % b\n    return a\n",
        [[12, 18], [7, 13], [0, 5]], [[100, 75], [17, 17], [48, 180]]),
    "Mbpp/10003": _task(
        "fibonacci", "fibonacci(n: int) -> int", "Return the n-th Fibonacci number with fibonacci(0) == 0 and fibonacci(1) == 1.",
        "    a, b = 0, 1\n    for _ in range(n):\n        a, b = b, a + b\n    return a\n",
        [[0], [1], [10]], [[2], [20], [30]]),
    "Mbpp/10004": _task(
        "is_prime", "is_prime(n: int) -> bool", "Return True iff n is a prime number.",
        "    if n < 2:\n        return False\n    i = 2\n    while i * i <= n:\n        if n % i == 0:\n            return False\n        i += 1\n    return True\n",
        [[2], [15], [17], [1]], [[0], [97], [100], [7919]]),
    "Mbpp/10005": _task(
        "running_max", "running_max(xs: list) -> list", "Return the list whose i-th element is max(xs[:i+1]).",
        "    out = []\n    for x in xs:\n        out.append(x if not out or x > out[-1] else out[-1])\n    return out\n",
        [[[1, 3, 2, 5, 4]], [[]], [[7]]], [[[5, 4, 3]], [[-1, -3, 0]]]),
    "Mbpp/10006": _task(
        "word_lengths", "word_lengths(s: str) -> list", "Return the lengths of the whitespace-separated words of s, in order.",
        "    return [len(w) for w in s.split()]\n",
        [["the quick brown fox"], [""], ["one"]], [["  padded   words "], ["a bb ccc"]]),
    "Mbpp/10007": _task(
        "mean", "mean(xs: list) -> float", "Arithmetic mean of a non-empty list of numbers.",
        "    return sum(xs) / len(xs)\n",
        [[[1, 2, 3]], [[2.5]], [[1, 2]]], [[[0.1, 0.2, 0.3]], [[-1, 1]]], atol=1e-9),
    "Mbpp/10008": _task(
        "chunk", "chunk(xs: list, n: int) -> list", "Split xs into consecutive pieces of length n (the last may be shorter).",
        "    return [xs[i:i + n] for i in range(0, len(xs), n)]\n",
        [[[1, 2, 3, 4, 5], 2], [[], 3], [[1, 2, 3], 3]], [[["a", "b", "c", "d"], 3], [[1], 5]]),
    "Mbpp/10009": _task(
        "digit_sum", "digit_sum(n: int) -> int", "Sum of the decimal digits of a non-negative integer.",
        "    return sum(int(c) for c in str(n))\n",
        [[0], [9], [123]], [[999], [1000001]]),
    "Mbpp/10010": _task(
        "invert_dict", "invert_dict(d: dict) -> dict", "Swap keys and values of a dict whose values are unique and hashable.",
        "    return {v: k for k, v in d.items()}\n",
        [[{"a": 1, "b": 2}], [{}]], [[{1: "x"}], [{"k": "v", "q": "w"}]]),
}
