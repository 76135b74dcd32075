from .cpp_tokenizer import (EXPECTED_SPECIAL_TOKENS, CppMegaTokenizer, TokenizerContractError, build_byte_fallback_tokenizer,
                            load_cppmega_tokenizer)
