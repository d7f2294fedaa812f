"""Reference arm of ``bench.py --impl reference``."""
import json


def main(args):
    print(json.dumps({"impl": "reference", "unavailable": "reference install not attempted yet"}), flush=True)
    return 0
