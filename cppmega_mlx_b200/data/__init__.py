from .batch import LMTokenBatch, ensure_lm_batch, synthetic_token_batch
from .fim import (FIM_SPECIAL_TOKEN_IDS, FIMSpecialTokenIds, apply_fim_permutation, apply_fim_transform,
                  apply_ifim_permutation, apply_ifim_transform, extract_ifim_instruction_text, sample_middle_span)
from .packing import (PackedSequences, cumulative_doc_ids_from_eos, document_boundary_mask, pack_bos_aligned_best_fit,
                      pack_documents_with_eos)
from .token_dataset import BatchCursor, TokenDatasetMetadata, TokenNpzDataset, iterate_token_batches, open_token_dataset
from .tokenizer_contract import REQUIRED_SPECIAL_TOKEN_IDS, validate_special_tokens
