// Open-addressing hash map from int32 keys to a trivially copyable value.
//
// Used for the child tables and endpoint tables of suffix-tree nodes, where the
// typical table holds one or two entries and the root holds up to a vocabulary's
// worth. Properties: power-of-two capacity, triangular probing (visits every
// slot), tombstones on erase, grow at 3/4 occupancy (live + tombstones), shrink
// when live entries fall under 1/8 of the capacity, 64-bit finaliser-style mix
// of the key. Up to two entries live inside the object itself: a map that small (most child
// and endpoint tables) owns no heap memory and is searched without hashing.
//
// Plays the role of csrc/suffix_decoding/int32_map.h in the reference.
#pragma once

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <new>
#include <utility>

namespace ab200 {

template <typename V>
class Int32Map {
 public:
  Int32Map() = default;
  Int32Map(const Int32Map&) = delete;
  Int32Map& operator=(const Int32Map&) = delete;
  Int32Map(Int32Map&& o) noexcept { steal(o); }
  Int32Map& operator=(Int32Map&& o) noexcept {
    if (this != &o) {
      release();
      steal(o);
    }
    return *this;
  }
  ~Int32Map() { release(); }

  uint32_t size() const { return cap_ == 0 ? in_ : live_; }
  bool empty() const { return size() == 0; }
  uint32_t capacity() const { return cap_; }
  size_t heap_bytes() const { return (size_t)cap_ * sizeof(Slot); }

  V* find(int32_t key) {
    if (cap_ == 0) {
      for (uint32_t i = 0; i < in_; ++i)
        if (ikey_[i] == key) return &ival_[i];
      return nullptr;
    }
    uint32_t i = mix(key) & (cap_ - 1);
    for (uint32_t step = 1;; ++step) {
      Slot& s = slots_[i];
      if (s.state == kEmpty) return nullptr;
      if (s.state == kFull && s.key == key) return &s.value;
      i = (i + step) & (cap_ - 1);
    }
  }
  const V* find(int32_t key) const { return const_cast<Int32Map*>(this)->find(key); }
  bool contains(int32_t key) const { return find(key) != nullptr; }

  // Insert or overwrite. Returns a reference to the stored value.
  V& put(int32_t key, const V& value) {
    if (cap_ == 0) {
      for (uint32_t i = 0; i < in_; ++i)
        if (ikey_[i] == key) {
          ival_[i] = value;
          return ival_[i];
        }
      if (in_ < kInline) {
        ikey_[in_] = key;
        ival_[in_] = value;
        return ival_[in_++];
      }
      spill();
    }
    if ((used_ + 1) * 4 > cap_ * 3) rehash(live_ + 1);
    uint32_t i = mix(key) & (cap_ - 1);
    int64_t grave = -1;
    for (uint32_t step = 1;; ++step) {
      Slot& s = slots_[i];
      if (s.state == kEmpty) break;
      if (s.state == kFull && s.key == key) {
        s.value = value;
        return s.value;
      }
      if (s.state == kTomb && grave < 0) grave = i;
      i = (i + step) & (cap_ - 1);
    }
    Slot& dst = grave >= 0 ? slots_[grave] : slots_[i];
    if (grave < 0) ++used_;
    dst.state = kFull;
    dst.key = key;
    dst.value = value;
    ++live_;
    return dst.value;
  }

  bool erase(int32_t key) {
    if (cap_ == 0) {
      for (uint32_t i = 0; i < in_; ++i)
        if (ikey_[i] == key) {
          --in_;
          ikey_[i] = ikey_[in_];
          ival_[i] = ival_[in_];
          return true;
        }
      return false;
    }
    uint32_t i = mix(key) & (cap_ - 1);
    for (uint32_t step = 1;; ++step) {
      Slot& s = slots_[i];
      if (s.state == kEmpty) return false;
      if (s.state == kFull && s.key == key) {
        s.state = kTomb;
        --live_;
        if (live_ == 0) {
          release();
        } else if (cap_ > kMinCap && live_ * 8 < cap_) {
          rehash(live_);
        }
        return true;
      }
      i = (i + step) & (cap_ - 1);
    }
  }

  void clear() { release(); }

  // Visit every (key, value); the callback must not modify the map.
  template <typename F>
  void for_each(F&& f) const {
    for (uint32_t i = 0; cap_ == 0 && i < in_; ++i) f(ikey_[i], ival_[i]);
    for (uint32_t i = 0; i < cap_; ++i)
      if (slots_[i].state == kFull) f(slots_[i].key, slots_[i].value);
  }

  // Any live entry (nullptr when empty).
  const std::pair<int32_t, V>* any(std::pair<int32_t, V>* scratch) const {
    if (cap_ == 0 && in_ > 0) {
      scratch->first = ikey_[0];
      scratch->second = ival_[0];
      return scratch;
    }
    for (uint32_t i = 0; i < cap_; ++i)
      if (slots_[i].state == kFull) {
        scratch->first = slots_[i].key;
        scratch->second = slots_[i].value;
        return scratch;
      }
    return nullptr;
  }

 private:
  enum : uint8_t { kEmpty = 0, kFull = 1, kTomb = 2 };
  static constexpr uint32_t kMinCap = 4;
  static constexpr uint32_t kInline = 2;
  struct Slot {
    int32_t key;
    uint8_t state;
    V value;
  };

  static uint32_t mix(int32_t key) {
    uint64_t z = (uint64_t)(uint32_t)key * 0x9E3779B97F4A7C15ull;
    z ^= z >> 32;
    z *= 0xD6E8FEB86659FD93ull;
    z ^= z >> 29;
    return (uint32_t)z;
  }

  void rehash(uint32_t want_live) {
    uint32_t cap = kMinCap;
    while (cap * 2 < want_live * 4 + 4) cap *= 2;  // target occupancy <= 1/2
    Slot* old = slots_;
    const uint32_t old_cap = cap_;
    slots_ = static_cast<Slot*>(std::calloc(cap, sizeof(Slot)));
    if (slots_ == nullptr) throw std::bad_alloc();
    cap_ = cap;
    used_ = 0;
    live_ = 0;
    for (uint32_t i = 0; i < old_cap; ++i)
      if (old[i].state == kFull) put_fresh(old[i].key, old[i].value);
    std::free(old);
  }

  void put_fresh(int32_t key, const V& value) {
    uint32_t i = mix(key) & (cap_ - 1);
    for (uint32_t step = 1; slots_[i].state != kEmpty; ++step) i = (i + step) & (cap_ - 1);
    slots_[i].state = kFull;
    slots_[i].key = key;
    slots_[i].value = value;
    ++used_;
    ++live_;
  }

  // the inline entries move to a freshly allocated table
  void spill() {
    const uint32_t n = in_;
    in_ = 0;
    slots_ = static_cast<Slot*>(std::calloc(8, sizeof(Slot)));
    if (slots_ == nullptr) throw std::bad_alloc();
    cap_ = 8;
    used_ = live_ = 0;
    for (uint32_t i = 0; i < n; ++i) put_fresh(ikey_[i], ival_[i]);
  }

  void release() {
    std::free(slots_);
    slots_ = nullptr;
    cap_ = used_ = live_ = 0;
    in_ = 0;
  }
  void steal(Int32Map& o) {
    slots_ = o.slots_;
    cap_ = o.cap_;
    used_ = o.used_;
    live_ = o.live_;
    in_ = o.in_;
    for (uint32_t i = 0; i < kInline; ++i) {
      ikey_[i] = o.ikey_[i];
      ival_[i] = o.ival_[i];
    }
    o.slots_ = nullptr;
    o.cap_ = o.used_ = o.live_ = 0;
    o.in_ = 0;
  }

  Slot* slots_ = nullptr;
  uint32_t cap_ = 0;
  uint32_t used_ = 0;  // full + tombstones
  uint32_t live_ = 0;
  uint32_t in_ = 0;    // inline entries in use (only while cap_ == 0)
  int32_t ikey_[kInline] = {};
  V ival_[kInline] = {};
};

}  // namespace ab200
