"""Imported once by the process that test ranks are forked from (``tests/dist_utils.py``): everything a rank would
otherwise import or initialise lazily on its own. The first ``torch.optim`` optimizer of a process pulls in several
hundred modules (the compiler stack behind ``torch.optim``'s decorators) and takes seconds; doing it here makes it a
one-time cost instead of a per-rank cost."""
import torch

import oslo_b200  # noqa: F401

torch.optim.AdamW([torch.nn.Parameter(torch.zeros(1))], lr=1e-3)
