from .io import (is_hf_safetensors_dir, load_checkpoint, model_state, resolve_checkpoint, save_checkpoint,
                 save_pretrained_dir)
from .name_maps import convert_name, framework_to_hf, fuse_state_dict, hf_to_framework, unfuse_state_dict, weight_dequant
from .resume import get_resume_checkpoint, record_resume_point, rescale_resume_step
from .transform import unify_checkpoints
