from .gpt2 import *  # noqa: F401,F403
from .gpt_neo import *  # noqa: F401,F403
from .gptj import *  # noqa: F401,F403
