from .adapter import (apply_lora, load_adapter, load_adapter_config, lora_state_dict, merge_adapter_into_base,
                      save_adapter, save_adapter_config)
