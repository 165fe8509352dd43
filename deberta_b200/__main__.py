"""``python -m deberta_b200`` → the unified CLI."""

from deberta_b200.cli import main

if __name__ == "__main__":
    main()
