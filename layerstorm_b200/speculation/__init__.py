from .combiner import DepthCalibrator, DraftCombiner, DraftSource, UtilityScorer, expected_tokens
from .dspark import DeviceDsparkDraft, DsparkBackbone, DsparkCheckpointConfig, DsparkDraft, DsparkScheduler, load_dspark_checkpoint
from .model_draft import ConfidenceHead, EngineDraft, MarkovHead, draft_shape_for
from .prompt_lookup import IncrementalPromptLookup, PromptLookupDraft
