"""The reference arm of bench.py: the unmodified reference through its own API."""
import json


def main(args, config, seed, point_prompt, prefill_tokens) -> int:
    print(json.dumps({"impl": "reference", "unavailable": "the reference arm is not set up yet"}))
    return 0
