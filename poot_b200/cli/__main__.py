"""``python -m poot_b200.cli generate -m CKPT -p "..." -n 16`` (crates/poot-llm/src/bin/poot/main.rs:42-55)."""
from __future__ import annotations

import sys

from .generate import main_generate

USAGE = "usage: poot {generate|caption|embed|plan} [options]   (generate --help lists the llama-cli compatible flags)"


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print(USAGE)
        return 0 if argv else 2
    cmd, rest = argv[0], argv[1:]
    if cmd == "generate":
        return main_generate(rest)
    if cmd == "embed":
        from .embed import main_embed
        return main_embed(rest)
    if cmd == "plan":
        from .plan import main_plan
        return main_plan(rest)
    if cmd == "caption":
        from .caption import main_caption
        return main_caption(rest)
    print(f"error: unknown command {cmd!r}\n{USAGE}", file=sys.stderr)
    return 2


if __name__ == "__main__":
    sys.exit(main())
