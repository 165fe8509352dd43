"""Entry point of ``python -m deberta_b200``: runs the command-line front end on the process arguments."""

from deberta_b200 import cli


def _run() -> int:
    cli.main()  # argv is read by the CLI itself (that is how it tells a real command line from a programmatic call)
    return 0


if __name__ == "__main__":
    raise SystemExit(_run())
