from .combiner import DepthCalibrator, DraftCombiner, DraftSource, UtilityScorer, expected_tokens
from .model_draft import ConfidenceHead, EngineDraft, MarkovHead, draft_shape_for
from .prompt_lookup import IncrementalPromptLookup, PromptLookupDraft
