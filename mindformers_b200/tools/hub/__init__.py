from .dynamic_module_utils import (check_imports, get_class_from_dynamic_module, get_class_in_module, get_imports,
                                   get_relative_imports, import_register_path)
from .hub import PushToHubMixin, create_repo, hf_hub_download, hub_root, repo_dir, snapshot_download, upload_folder
