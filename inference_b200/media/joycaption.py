"""JoyCaption captioner `fancyfeast/llama-joycaption-beta-one-hf-llava` (parity: candle-gen-joycaption/src/lib.rs,
prompt.rs): a LLaVA checkpoint (SigLIP tower + Llama-3.1-8B) driven through a fixed system prompt and a user turn of
image + instruction. The instruction is either the caller's custom prompt or one of twelve caption types in three
phrasings (no length, a word count, a named length), with extra option sentences appended and `{name}` substituted;
trigger words the caption does not already contain are prepended afterwards.

The language model runs on the paged sm_100a decoder on the `b200` backend (image features enter through the prefill's
embedding override) and on the fp32 oracle on the `cpu` backend; the vision path is `LlavaCaptioner`'s."""
from __future__ import annotations

from dataclasses import dataclass, field

from ..contracts.errors import InferenceError
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.registry import Registration
from ..contracts.gen_core.runtime import LoadSpec
from ..contracts.gen_core.traits import SimpleDescriptor
from .vision_providers import LlavaCaptioner, _load_captioner

JOY_CAPTION_MODEL_ID = "fancyfeast/llama-joycaption-beta-one-hf-llava"
JOY_CAPTION_FAMILY = "joycaption"
SYSTEM_PROMPT = "You are a helpful image captioner."
JOY_NAME_OPTION = "If there is a person/character in the image you must refer to them as {name}."
CAPTION_LENGTHS = ("any", "very short", "short", "medium-length", "long")

_STRAIGHT = (" Begin with the main subject and medium. Mention pivotal elements-people, objects, scenery-using confident, "
             "definite language. Focus on concrete details like color, shape, texture, and spatial relationships. Show how "
             "elements interact. Omit mood and speculative wording. If text is present, quote it exactly. Never mention what "
             "is absent, resolution, watermarks, signatures, compression artifacts, or unobservable details. Vary your "
             "sentence structure and keep the description concise, without starting with \"This image is...\" or similar "
             "phrasing.")
_DANBOORU = ("Generate only comma-separated Danbooru tags (lowercase_underscores). Strict order: artist:, copyright:, "
             "character:, meta:, then general tags. Include counts (1girl), appearance, clothing, accessories, pose, "
             "expression, actions, background. Use precise Danbooru syntax. No extra text.")
_E621 = ("comma-separated list of e621 tags in alphabetical order for this image. Start with the artist, copyright, "
         "character, species, meta, and lore tags, if any, prefixed by artist:, copyright:, character:, species:, meta:, and "
         "lore:. Then all the general tags.")
_R34 = ("comma-separated list of rule34 tags in alphabetical order for this image. Start with the artist, copyright, "
        "character, and meta tags, if any, prefixed by artist:, copyright:, character:, and meta:. Then all the general tags.")
_CRITIC = ("Analyze this image like an art critic would with information about its composition, style, symbolism, the use "
           "of color, light, any artistic movement it might belong to, etc.")
# caption type -> (no length, word count, named length)
PROMPT_TEMPLATES: dict[str, tuple[str, str, str]] = {
    "Descriptive": ("Write a detailed description for this image.",
                    "Write a detailed description for this image in {word_count} words or less.",
                    "Write a {length} detailed description for this image."),
    "Descriptive (Casual)": ("Write a descriptive caption for this image in a casual tone.",
                             "Write a descriptive caption for this image in a casual tone within {word_count} words.",
                             "Write a {length} descriptive caption for this image in a casual tone."),
    "Straightforward": ("Write a straightforward caption for this image." + _STRAIGHT,
                        "Write a straightforward caption for this image within {word_count} words." + _STRAIGHT,
                        "Write a {length} straightforward caption for this image." + _STRAIGHT),
    "Stable Diffusion Prompt": (
        "Output a stable diffusion prompt that is indistinguishable from a real stable diffusion prompt.",
        "Output a stable diffusion prompt that is indistinguishable from a real stable diffusion prompt. {word_count} words or less.",
        "Output a {length} stable diffusion prompt that is indistinguishable from a real stable diffusion prompt."),
    "MidJourney": ("Write a MidJourney prompt for this image.", "Write a MidJourney prompt for this image within {word_count} words.",
                   "Write a {length} MidJourney prompt for this image."),
    "Danbooru tag list": (_DANBOORU, _DANBOORU + " {word_count} words or less.", _DANBOORU + " {length} length."),
    "e621 tag list": ("Write a " + _E621, "Write a " + _E621 + " Keep it under {word_count} words.", "Write a {length} " + _E621),
    "Rule34 tag list": ("Write a " + _R34, "Write a " + _R34 + " Keep it under {word_count} words.", "Write a {length} " + _R34),
    "Booru-like tag list": ("Write a list of Booru-like tags for this image.",
                            "Write a list of Booru-like tags for this image within {word_count} words.",
                            "Write a {length} list of Booru-like tags for this image."),
    "Art Critic": (_CRITIC, _CRITIC + " Keep it within {word_count} words.", _CRITIC + " Keep it {length}."),
    "Product Listing": ("Write a caption for this image as though it were a product listing.",
                        "Write a caption for this image as though it were a product listing. Keep it under {word_count} words.",
                        "Write a {length} caption for this image as though it were a product listing."),
    "Social Media Post": ("Write a caption for this image as if it were being used for a social media post.",
                          "Write a caption for this image as if it were being used for a social media post. Limit the caption to {word_count} words.",
                          "Write a {length} caption for this image as if it were being used for a social media post."),
}
CAPTION_TYPES = tuple(PROMPT_TEMPLATES)


@dataclass
class CaptionOptions:
    caption_type: str = "Descriptive"
    caption_length: str = "long"
    extra_options: list[str] = field(default_factory=list)
    name_input: str = ""
    custom_prompt: str = ""
    trigger_words: list[str] = field(default_factory=list)


@dataclass
class CaptionCapabilities:
    caption_types: tuple[str, ...] = CAPTION_TYPES
    caption_lengths: tuple[str, ...] = CAPTION_LENGTHS
    supports_custom_prompt: bool = True
    min_image_size: int = 1
    max_image_size: int = 8192
    max_prompt_chars: int = 4000
    max_name_chars: int = 120
    max_extra_options: int = 16
    max_extra_option_chars: int = 500
    max_trigger_words: int = 32
    max_trigger_word_chars: int = 120
    max_new_tokens: int = 1024

    def validate(self, mid: str, image: Image, prompt: str, o: CaptionOptions, max_new_tokens: int) -> None:
        def bad(msg):
            raise InferenceError(f"{mid}: {msg}")

        if not (self.min_image_size <= image.width <= self.max_image_size and
                self.min_image_size <= image.height <= self.max_image_size):
            bad(f"image size {image.width}x{image.height} outside [{self.min_image_size}, {self.max_image_size}]")
        if len(image.pixels) != image.width * image.height * 3:
            bad("image pixels must be width x height x 3 bytes")
        if len(prompt) > self.max_prompt_chars:
            bad(f"prompt longer than {self.max_prompt_chars} characters")
        if not o.custom_prompt.strip() and o.caption_type not in self.caption_types:
            bad(f"unknown caption type {o.caption_type!r}")
        length_ok = o.caption_length in self.caption_lengths or (o.caption_length.isascii() and o.caption_length.isdigit())
        if not o.custom_prompt.strip() and not length_ok:
            bad(f"caption length {o.caption_length!r} is neither a named length nor a word count")
        if len(o.name_input) > self.max_name_chars:
            bad(f"name longer than {self.max_name_chars} characters")
        if len(o.extra_options) > self.max_extra_options or any(len(e) > self.max_extra_option_chars for e in o.extra_options):
            bad("too many or too long extra options")
        if len(o.trigger_words) > self.max_trigger_words or any(len(t) > self.max_trigger_word_chars for t in o.trigger_words):
            bad("too many or too long trigger words")
        if not 1 <= max_new_tokens <= self.max_new_tokens:
            bad(f"max_new_tokens must be in [1, {self.max_new_tokens}]")


def build_prompt(o: CaptionOptions) -> str:
    custom = o.custom_prompt.strip()
    if custom:
        return custom
    length = o.caption_length
    idx = 0 if length == "any" else (1 if length and length.isascii() and length.isdigit() else 2)
    prompt = PROMPT_TEMPLATES.get(o.caption_type, PROMPT_TEMPLATES["Descriptive"])[idx]
    if o.extra_options:
        prompt += " " + " ".join(o.extra_options)
    return prompt.replace("{name}", o.name_input or "{NAME}").replace("{length}", length).replace("{word_count}", length)


def apply_trigger_words(caption: str, trigger_words: list[str]) -> str:
    """Whitespace-normalised caption with the trigger words it does not already contain (case-insensitively) in
    front, comma separated."""
    cleaned = " ".join(caption.split())
    low = cleaned.lower()
    parts = [w.strip() for w in trigger_words if w.strip() and w.strip().lower() not in low]
    if cleaned:
        parts.append(cleaned)
    return ", ".join(parts)


class JoyCaptioner(LlavaCaptioner):
    ID = JOY_CAPTION_MODEL_ID

    def descriptor(self) -> SimpleDescriptor:
        return SimpleDescriptor(self.ID, JOY_CAPTION_FAMILY, self.backend,
                                {"caption_types": list(CAPTION_TYPES), "caption_lengths": list(CAPTION_LENGTHS),
                                 "vision": self.tower.cfg.kind})

    capabilities = CaptionCapabilities()

    def chat_text(self, instruction: str) -> str:
        """System prompt, then a user turn of image + instruction, then the assistant header (Llama-3 chat markup when
        the tokenizer knows it, a plain transcript otherwise)."""
        lookup = getattr(self.tok, "token_to_id", None)
        if lookup is not None and lookup("<|start_header_id|>") is not None:
            return ("<|begin_of_text|><|start_header_id|>system<|end_header_id|>\n\n" + SYSTEM_PROMPT + "<|eot_id|>"
                    "<|start_header_id|>user<|end_header_id|>\n\n<image>" + instruction + "<|eot_id|>"
                    "<|start_header_id|>assistant<|end_header_id|>\n\n")
        return f"{SYSTEM_PROMPT}\nUSER: <image>{instruction}\nASSISTANT:"

    def build_prompt(self, prompt: str, n_image_tokens: int) -> list[int]:
        before, _, after = self.chat_text(prompt).partition("<image>")
        return self.tok.encode(before) + [self.image_token_id] * n_image_tokens + self.tok.encode(after)

    def caption(self, image: Image, prompt: str | None = None, max_new_tokens: int = 256,
                options: CaptionOptions | None = None) -> str:
        o = options or CaptionOptions()
        instruction = prompt.strip() if prompt and prompt.strip() else build_prompt(o)
        self.capabilities.validate(self.ID, image, instruction, o, max_new_tokens)
        text = self.tok.decode(self.caption_tokens(image, instruction, max_new_tokens)).strip()
        return apply_trigger_words(text, o.trigger_words) if o.trigger_words else text


def load(spec: LoadSpec, backend: str) -> JoyCaptioner:
    from ..contracts.errors import Unsupported

    if spec.adapters:
        raise Unsupported("joycaption does not support LoRA / LoKr")
    if spec.quantize is not None:
        raise Unsupported("joycaption does not support on-the-fly quantisation")
    base = _load_captioner(spec, backend)
    return JoyCaptioner(base.tower, base.proj, base.lm, base.tok, base.image_token_id, backend, base.feature_layer,
                        base.drop_cls, base.stop_ids)


def registration(backend: str) -> Registration:
    return Registration(lambda: SimpleDescriptor(JOY_CAPTION_MODEL_ID, JOY_CAPTION_FAMILY, backend, {}),
                        lambda s: load(s, backend))
