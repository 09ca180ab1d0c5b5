"""Audio feature extraction on numpy arrays: mel scales, triangular filter banks, window functions, short-time Fourier
spectrograms and decibel conversion.

API counterpart of the reference's ``dataset/transforms/audio_utils.py`` (``hertz_to_mel`` :26, ``mel_to_hertz`` :62,
``mel_filter_bank`` :218, ``optimal_fft_length`` :306, ``window_function`` :319, ``spectrogram`` :382, ``power_to_db``
:793, ``amplitude_to_db`` :893), written from the definitions:

* mel scales: ``htk``  m = 2595 log10(1 + f / 700);  ``kaldi``  m = 1127 ln(1 + f / 700);  ``slaney``  linear below
  1 kHz (3 mel per 200 Hz) and logarithmic above (27 steps per factor 6.4);
* a mel filter bank is a set of triangles whose corner frequencies are equally spaced on the mel scale; ``norm="slaney"``
  scales every triangle to unit area;
* the spectrogram frames the (optionally centre-padded, pre-emphasised) waveform, applies the window, takes the real
  FFT and raises the magnitude to ``power``; mel filters and a log are applied on request.
"""
from __future__ import annotations

from typing import Optional, Union

import numpy as np

_SLANEY_BREAK_HZ = 1000.0
_SLANEY_BREAK_MEL = 15.0
_SLANEY_LOGSTEP = 27.0 / np.log(6.4)


def hertz_to_mel(freq: Union[float, np.ndarray], mel_scale: str = "htk") -> Union[float, np.ndarray]:
    if mel_scale not in ("htk", "kaldi", "slaney"):
        raise ValueError('mel_scale should be one of "htk", "slaney" or "kaldi".')
    f = np.asarray(freq, dtype=np.float64)
    if mel_scale == "htk":
        out = 2595.0 * np.log10(1.0 + f / 700.0)
    elif mel_scale == "kaldi":
        out = 1127.0 * np.log(1.0 + f / 700.0)
    else:
        lin = 3.0 * f / 200.0
        with np.errstate(divide="ignore", invalid="ignore"):
            log = _SLANEY_BREAK_MEL + np.log(np.maximum(f, 1e-300) / _SLANEY_BREAK_HZ) * _SLANEY_LOGSTEP
        out = np.where(f >= _SLANEY_BREAK_HZ, log, lin)
    return float(out) if np.isscalar(freq) else out


def mel_to_hertz(mels: Union[float, np.ndarray], mel_scale: str = "htk") -> Union[float, np.ndarray]:
    if mel_scale not in ("htk", "kaldi", "slaney"):
        raise ValueError('mel_scale should be one of "htk", "slaney" or "kaldi".')
    m = np.asarray(mels, dtype=np.float64)
    if mel_scale == "htk":
        out = 700.0 * (np.power(10.0, m / 2595.0) - 1.0)
    elif mel_scale == "kaldi":
        out = 700.0 * (np.exp(m / 1127.0) - 1.0)
    else:
        lin = 200.0 * m / 3.0
        log = _SLANEY_BREAK_HZ * np.exp((m - _SLANEY_BREAK_MEL) / _SLANEY_LOGSTEP)
        out = np.where(m >= _SLANEY_BREAK_MEL, log, lin)
    return float(out) if np.isscalar(mels) else out


def _triangles(fft_freqs: np.ndarray, corners: np.ndarray) -> np.ndarray:
    """``[num_bins, num_filters]``: filter j rises from corner j to j + 1 and falls to j + 2."""
    widths = np.diff(corners)
    offset = corners[None, :] - fft_freqs[:, None]                 # [bins, filters + 2]
    rising = -offset[:, :-2] / widths[:-1]
    falling = offset[:, 2:] / widths[1:]
    return np.maximum(0.0, np.minimum(rising, falling))


def mel_filter_bank(num_frequency_bins: int, num_mel_filters: int, min_frequency: float, max_frequency: float,
                    sampling_rate: int, norm: Optional[str] = None, mel_scale: str = "htk",
                    triangularize_in_mel_space: bool = False) -> np.ndarray:
    """``[num_frequency_bins, num_mel_filters]`` projection from FFT bins to mel bands."""
    if norm is not None and norm != "slaney":
        raise ValueError('norm must be one of None or "slaney"')
    mel_lo, mel_hi = hertz_to_mel(min_frequency, mel_scale), hertz_to_mel(max_frequency, mel_scale)
    mel_pts = np.linspace(mel_lo, mel_hi, num_mel_filters + 2)
    corners_hz = mel_to_hertz(mel_pts, mel_scale)
    if triangularize_in_mel_space:
        bin_width = sampling_rate / (2.0 * (num_frequency_bins - 1))
        bins = hertz_to_mel(bin_width * np.arange(num_frequency_bins), mel_scale)
        bank = _triangles(bins, mel_pts)
    else:
        bins = np.linspace(0.0, sampling_rate // 2, num_frequency_bins)
        bank = _triangles(bins, corners_hz)
    if norm == "slaney":
        bank = bank * (2.0 / (corners_hz[2:] - corners_hz[:-2]))[None, :]
    return bank


def optimal_fft_length(window_length: int) -> int:
    """The next power of two: the FFT size for a window of ``window_length`` samples."""
    return 1 << max(0, int(window_length) - 1).bit_length()


def window_function(window_length: int, name: str = "hann", periodic: bool = True, frame_length: Optional[int] = None,
                    center: bool = True) -> np.ndarray:
    """``boxcar``, ``hann`` (``hann_window``), ``hamming`` (``hamming_window``) or ``povey`` (hann ** 0.85); a periodic
    window is the symmetric window of one more sample without its last point. With ``frame_length`` the window is
    zero-padded (centred or left-aligned) to that length."""
    n = window_length + 1 if periodic else window_length
    k = np.arange(n)
    if name == "boxcar":
        w = np.ones(n)
    elif name in ("hamming", "hamming_window"):
        w = 0.54 - 0.46 * np.cos(2 * np.pi * k / max(n - 1, 1))
    elif name in ("hann", "hann_window"):
        w = 0.5 - 0.5 * np.cos(2 * np.pi * k / max(n - 1, 1))
    elif name == "povey":
        w = np.power(0.5 - 0.5 * np.cos(2 * np.pi * k / max(n - 1, 1)), 0.85)
    else:
        raise ValueError(f"Unknown window function '{name}'")
    if periodic:
        w = w[:-1]
    if frame_length is None:
        return w
    if window_length > frame_length:
        raise ValueError(f"Length of the window ({window_length}) may not be larger than frame_length ({frame_length})")
    out = np.zeros(frame_length)
    off = (frame_length - window_length) // 2 if center else 0
    out[off:off + window_length] = w
    return out


def power_to_db(spectrogram_: np.ndarray, reference: float = 1.0, min_value: float = 1e-10,
                db_range: Optional[float] = None) -> np.ndarray:
    """``10 log10(S / reference)`` with ``S`` clipped below at ``min_value``; ``db_range`` limits the dynamic range below
    the maximum."""
    if reference <= 0.0:
        raise ValueError("reference must be greater than zero")
    if min_value <= 0.0:
        raise ValueError("min_value must be greater than zero")
    s = np.clip(np.asarray(spectrogram_, dtype=np.float64), a_min=min_value, a_max=None)
    out = 10.0 * (np.log10(s) - np.log10(max(min_value, reference)))
    if db_range is not None:
        if db_range <= 0.0:
            raise ValueError("db_range must be greater than zero")
        out = np.clip(out, a_min=out.max() - db_range, a_max=None)
    return out


def amplitude_to_db(spectrogram_: np.ndarray, reference: float = 1.0, min_value: float = 1e-5,
                    db_range: Optional[float] = None) -> np.ndarray:
    """``20 log10(A / reference)``: the decibel value of an amplitude spectrogram."""
    if reference <= 0.0:
        raise ValueError("reference must be greater than zero")
    if min_value <= 0.0:
        raise ValueError("min_value must be greater than zero")
    s = np.clip(np.asarray(spectrogram_, dtype=np.float64), a_min=min_value, a_max=None)
    out = 20.0 * (np.log10(s) - np.log10(max(min_value, reference)))
    if db_range is not None:
        if db_range <= 0.0:
            raise ValueError("db_range must be greater than zero")
        out = np.clip(out, a_min=out.max() - db_range, a_max=None)
    return out


def spectrogram(waveform: np.ndarray, window: np.ndarray, frame_length: int, hop_length: int,
                fft_length: Optional[int] = None, power: Optional[float] = 1.0, center: bool = True,
                pad_mode: str = "reflect", onesided: bool = True, preemphasis: Optional[float] = None,
                mel_filters: Optional[np.ndarray] = None, mel_floor: float = 1e-10, log_mel: Optional[str] = None,
                reference: float = 1.0, min_value: float = 1e-10, db_range: Optional[float] = None,
                remove_dc_offset: bool = False, dtype=np.float32) -> np.ndarray:
    """``[num_frequency_bins (or mel bands), num_frames]`` spectrogram of a mono waveform.

    ``power`` 1 gives amplitudes, 2 energies, None the complex STFT. ``log_mel``: ``"log"`` (natural), ``"log10"`` or
    ``"dB"`` (``power_to_db`` for power 2, ``amplitude_to_db`` for power 1)."""
    waveform = np.asarray(waveform)
    if waveform.ndim != 1:
        raise ValueError(f"Input waveform must have only one dimension, shape is {waveform.shape}")
    if np.iscomplexobj(waveform):
        raise ValueError("Complex-valued input waveforms are not currently supported")
    window = np.asarray(window, dtype=np.float64)
    if len(window) != frame_length:
        raise ValueError(f"Length of the window ({len(window)}) must equal frame_length ({frame_length})")
    fft_length = fft_length or frame_length
    if frame_length > fft_length:
        raise ValueError(f"frame_length ({frame_length}) may not be larger than fft_length ({fft_length})")
    if hop_length <= 0:
        raise ValueError("hop_length must be greater than zero")
    if power is None and mel_filters is not None:
        raise ValueError("You have provided `mel_filters` but `power` is `None`: mel filters need a real spectrogram")
    x = waveform.astype(np.float64)
    if center:
        x = np.pad(x, (frame_length // 2, frame_length // 2), mode=pad_mode)
    n_frames = int(1 + (len(x) - frame_length) // hop_length) if len(x) >= frame_length else 0
    idx = np.arange(frame_length)[None, :] + hop_length * np.arange(n_frames)[:, None]
    frames = x[idx] if n_frames else np.zeros((0, frame_length))
    if remove_dc_offset:
        frames = frames - frames.mean(axis=1, keepdims=True)
    if preemphasis is not None:
        shifted = np.concatenate([frames[:, :1], frames[:, :-1]], axis=1)
        frames = frames - preemphasis * shifted
    frames = frames * window[None, :]
    spec = (np.fft.rfft(frames, n=fft_length, axis=1) if onesided else np.fft.fft(frames, n=fft_length, axis=1)).T
    if power is not None:
        spec = np.abs(spec) ** power
    if mel_filters is not None:
        spec = np.maximum(mel_floor, mel_filters.T @ spec)
    if power is not None and log_mel is not None:
        if log_mel == "log":
            spec = np.log(spec)
        elif log_mel == "log10":
            spec = np.log10(spec)
        elif log_mel == "dB":
            if power == 1.0:
                spec = amplitude_to_db(spec, reference, min_value, db_range)
            elif power == 2.0:
                spec = power_to_db(spec, reference, min_value, db_range)
            else:
                raise ValueError(f"Cannot use log_mel option '{log_mel}' with power {power}")
        else:
            raise ValueError(f"Unknown log_mel option: {log_mel}")
    return np.asarray(spec, dtype=dtype if power is not None else np.complex64)
