# SPDX-License-Identifier: MIT
"""`barlink_sm86`: the reference's import name, kept so that code written
against it (`import barlink_sm86 as bl`, `from barlink_sm86 import
process_group`) finds the same op surface (torch_ext/barlink_sm86/__init__.py:
62-73).  Everything is implemented in `barlink_sm86_b200`."""
import sys

import barlink_sm86_b200 as _impl
from barlink_sm86_b200 import *  # noqa: F401,F403
from barlink_sm86_b200 import _C, process_group  # noqa: F401

sys.modules.setdefault(__name__ + ".process_group", process_group)
__all__ = list(_impl.__all__)
