from .base_model import (BaseXModalToTextModel, ImageToTextConfig, ImageToTextModel, VisionConfig, ViTEncoder)
from .base_processor import (BaseImageProcessor, BaseImageToTextImageProcessor, BaseXModalToTextProcessor,
                             BaseXModalToTextTransform)
from .modal_content import (BaseImageContentBuilder, BaseTextContentBuilder, DataRecord, ModalContentBuilder,
                            ModalContentTransformTemplate)
