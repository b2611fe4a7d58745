from .beam_search import BeamHypotheses, BeamSearchScorer  # noqa: F401
from .logits_process import *  # noqa: F401,F403
from .utils import GenerateOutput, GenerationMixin  # noqa: F401
from .graph_decode import GraphedGreedyDecoder  # noqa: F401
