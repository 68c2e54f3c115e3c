from .loss import CrossTokenizerDistillationLossFn
from .token_aligner import TokenAligner, build_vocab_projection
