# SPDX-License-Identifier: MIT
"""`python -m barlink_sm86._bootstrap script.py ...` -- same entry as the
reference's bootstrap module; see barlink_sm86_b200/_bootstrap.py."""
from barlink_sm86_b200._bootstrap import main

if __name__ == "__main__":
    main()
