"""What the command-line entry points share: an input problem (a missing file, a malformed model or shard, a bad value) ends a
command with one line on stderr and exit status 2, not with a traceback.  ``B200_TRACEBACK=1`` keeps the traceback."""
from __future__ import annotations

import functools
import os
import sys


def cli_entry(prog: str):
    """Wrap ``main(argv=None)``.  Only a real command-line run (``argv`` is None) is translated; a caller that passes ``argv``
    itself (a test, another program) gets the exception."""

    def deco(main):
        @functools.wraps(main)
        def run(argv=None):
            if argv is not None or os.environ.get("B200_TRACEBACK") == "1":
                return main(argv)
            try:
                return main(argv)
            except KeyboardInterrupt:
                sys.stderr.write(f"{prog}: interrupted\n")
                raise SystemExit(130)
            except (OSError, ValueError) as e:     # ValueError covers malformed files, JSON and argument values
                what = f"{e.filename}: {e.strerror}" if isinstance(e, OSError) and e.filename else (str(e) or type(e).__name__)
                sys.stderr.write(f"{prog}: error: {what}\n")
                raise SystemExit(2)
        return run
    return deco
