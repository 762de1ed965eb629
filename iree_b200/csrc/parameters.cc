// Parameter archives (.irpa): index, writer, and loading of parameters into device memory.
//
// The file format is the reference's (runtime/src/iree/schemas/parameter_archive.h:1-241): a
// 16-byte aligned header chain; each v0 header points at an entry table (16-byte aligned
// entries: splat / data / external), a metadata segment holding the names, and a storage segment
// holding the bytes of data entries. The index mirrors iree_io_parameter_index_t
// (runtime/src/iree/io/parameter_index.h), the parser iree_io_parse_irpa_index
// (io/formats/irpa/irpa_parser.c:150-348, same checks and status codes), the writer
// iree_io_parameter_archive_builder_* (io/formats/irpa/irpa_builder.c:46-330, same layout, so
// archives are byte-identical to the ones the reference's iree-create-parameters writes), and
// loading does what iree_io_parameter_index_provider's load / gather does for a HAL buffer
// (io/parameter_index_provider.c): file-backed entries are copied host -> device, splats are
// filled on the device.
#include <errno.h>
#include <fcntl.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <string>
#include <vector>

#include "../../include/iree_b200.h"
#include "hal_b200_internal.h"

namespace {

iree_b200_status_t pfail(iree_b200_status_t code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  return static_cast<iree_b200_status_t>(iree_b200_internal_set_error(code, buf));
}

// On-disk structures (packed, little-endian), parameter_archive.h:60-235.
#pragma pack(push, 1)
struct Range {
  uint64_t offset, length;
};
struct HeaderPrefix {
  uint32_t magic;
  uint16_t version_major, version_minor;
  uint64_t header_size, next_header_offset, flags;
};
struct HeaderV0 {
  HeaderPrefix prefix;
  uint64_t entry_count;
  Range entry_segment, metadata_segment, storage_segment;
};
struct EntryHeader {
  uint64_t entry_size;
  uint32_t type;
  uint64_t flags;
  Range name, metadata;
  uint64_t minimum_alignment;
};
struct SplatEntry {
  EntryHeader header;
  uint64_t length;
  uint8_t pattern[16];
  uint8_t pattern_length;
};
struct DataEntry {
  EntryHeader header;
  Range storage;
};
#pragma pack(pop)
static_assert(sizeof(HeaderPrefix) == 32 && sizeof(HeaderV0) == 88, "header layout");
static_assert(sizeof(EntryHeader) == 60 && sizeof(SplatEntry) == 85 && sizeof(DataEntry) == 76, "entry layout");

constexpr uint32_t kMagic = 0x41505249u;  // "IRPA"
constexpr uint64_t kHeaderAlignment = 16, kEntryAlignment = 16, kFileAlignment = 4096;
enum : uint32_t { kEntrySkip = 0, kEntrySplat = 1, kEntryData = 2, kEntryExternal = 3 };

uint64_t align_up(uint64_t v, uint64_t a) { return a ? (v + a - 1) / a * a : v; }

struct Entry {
  std::string key, metadata;
  uint64_t length = 0;
  int32_t type = IREE_B200_PARAMETER_STORAGE_FILE;
  uint8_t pattern[16] = {0};
  uint8_t pattern_length = 0;
  uint64_t file_offset = 0;  // absolute, file-backed entries
};

}  // namespace

struct iree_b200_parameter_index_t {
  std::vector<Entry> entries;
  // the mapped archive (file-backed entries point into it)
  const uint8_t* base = nullptr;
  size_t size = 0;
  int fd = -1;
  bool owns_mapping = false;
};

namespace {

iree_b200_status_t verify_range(uint64_t base, Range r, uint64_t file_size) {
  const uint64_t begin = base + r.offset, end = begin + r.length;
  if (begin > file_size || end > file_size || end < begin)
    return pfail(IREE_B200_STATUS_OUT_OF_RANGE, "file segment out of range (%llu to %llu for %llu, file_size=%llu)",
                 (unsigned long long)begin, (unsigned long long)end, (unsigned long long)r.length,
                 (unsigned long long)file_size);
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t resolve_metadata(const uint8_t* file, uint64_t base, Range segment, Range ref, std::string* out) {
  out->clear();
  if (ref.length == 0) return IREE_B200_STATUS_OK;
  const uint64_t end = ref.offset + ref.length;
  if (ref.offset > segment.length || end > segment.length || end < ref.offset)
    return pfail(IREE_B200_STATUS_OUT_OF_RANGE,
                 "metadata segment reference out of range (%llu to %llu for %llu, segment_size=%llu)",
                 (unsigned long long)ref.offset, (unsigned long long)end, (unsigned long long)ref.length,
                 (unsigned long long)segment.length);
  out->assign(reinterpret_cast<const char*>(file + base + segment.offset + ref.offset), ref.length);
  return IREE_B200_STATUS_OK;
}

// One v0 header and its entry table (irpa_parser.c:150-262).
iree_b200_status_t parse_header_v0(const uint8_t* file, uint64_t file_size, uint64_t base, const HeaderPrefix& prefix,
                                   iree_b200_parameter_index_t* index) {
  if (prefix.version_minor > 0)
    return pfail(IREE_B200_STATUS_UNIMPLEMENTED,
                 "IRPA version %u.%u not supported (major supported but minor is newer than the runtime trying to parse it)",
                 prefix.version_major, prefix.version_minor);
  if (prefix.header_size != sizeof(HeaderV0))
    return pfail(IREE_B200_STATUS_INVALID_ARGUMENT, "IRPA v0 header expected to be exactly %zu bytes but was reported as %llu",
                 sizeof(HeaderV0), (unsigned long long)prefix.header_size);
  HeaderV0 h;
  memcpy(&h, file + base, sizeof h);
  if (iree_b200_status_t st = verify_range(base, h.entry_segment, file_size)) return st;
  if (iree_b200_status_t st = verify_range(base, h.metadata_segment, file_size)) return st;
  if (iree_b200_status_t st = verify_range(base, h.storage_segment, file_size)) return st;
  uint64_t offset = 0;
  for (uint64_t i = 0; i < h.entry_count; ++i) {
    offset = align_up(offset, kEntryAlignment);
    if (offset + sizeof(EntryHeader) > h.entry_segment.length)
      return pfail(IREE_B200_STATUS_OUT_OF_RANGE, "entry table truncated; insufficient bytes for base entry header");
    EntryHeader eh;
    memcpy(&eh, file + base + h.entry_segment.offset + offset, sizeof eh);
    if (eh.entry_size < sizeof(EntryHeader) || offset + eh.entry_size > h.entry_segment.length)
      return pfail(IREE_B200_STATUS_OUT_OF_RANGE, "entry table truncated; insufficient bytes for sized header");
    const uint8_t* raw = file + base + h.entry_segment.offset + offset;
    offset += eh.entry_size;
    if (eh.type == kEntrySkip) continue;
    Entry e;
    if (iree_b200_status_t st = resolve_metadata(file, base, h.metadata_segment, eh.name, &e.key)) return st;
    if (iree_b200_status_t st = resolve_metadata(file, base, h.metadata_segment, eh.metadata, &e.metadata)) return st;
    if (eh.type == kEntrySplat) {
      if (eh.entry_size < sizeof(SplatEntry)) return pfail(IREE_B200_STATUS_OUT_OF_RANGE, "splat entry length underflow");
      SplatEntry s;
      memcpy(&s, raw, sizeof s);
      if (s.pattern_length > sizeof s.pattern)
        return pfail(IREE_B200_STATUS_INVALID_ARGUMENT, "splat pattern length %u out of bounds %zu", s.pattern_length,
                     sizeof s.pattern);
      e.type = IREE_B200_PARAMETER_STORAGE_SPLAT;
      e.length = s.length;
      e.pattern_length = s.pattern_length;
      memcpy(e.pattern, s.pattern, sizeof e.pattern);
    } else if (eh.type == kEntryData) {
      if (eh.entry_size < sizeof(DataEntry)) return pfail(IREE_B200_STATUS_OUT_OF_RANGE, "data entry length underflow");
      DataEntry d;
      memcpy(&d, raw, sizeof d);
      const uint64_t end = d.storage.offset + d.storage.length;
      if (d.storage.offset > h.storage_segment.length || end > h.storage_segment.length || end < d.storage.offset)
        return pfail(IREE_B200_STATUS_OUT_OF_RANGE,
                     "storage segment reference out of range (%llu to %llu for %llu, segment_size=%llu)",
                     (unsigned long long)d.storage.offset, (unsigned long long)end, (unsigned long long)d.storage.length,
                     (unsigned long long)h.storage_segment.length);
      e.type = IREE_B200_PARAMETER_STORAGE_FILE;
      e.length = d.storage.length;
      e.file_offset = base + h.storage_segment.offset + d.storage.offset;
    } else {
      return pfail(IREE_B200_STATUS_UNIMPLEMENTED, "parser does not support entry type %d", (int)eh.type);
    }
    index->entries.push_back(std::move(e));
  }
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t parse_archive(const uint8_t* file, uint64_t file_size, iree_b200_parameter_index_t* index) {
  uint64_t base = 0;
  while (true) {
    if (file_size < base + sizeof(HeaderPrefix))
      return pfail(IREE_B200_STATUS_INVALID_ARGUMENT,
                   "not enough bytes for a valid IRPA header; file may be empty or truncated");
    HeaderPrefix prefix;
    memcpy(&prefix, file + base, sizeof prefix);
    if (prefix.magic != kMagic)
      return pfail(IREE_B200_STATUS_INVALID_ARGUMENT, "IRPA file magic missing or invalid %08X; expected %08X", prefix.magic,
                   kMagic);
    if (base + prefix.header_size > file_size || base + prefix.header_size < base)
      return pfail(IREE_B200_STATUS_OUT_OF_RANGE,
                   "file buffer underrun parsing header of reported size %llu (only %llu bytes available)",
                   (unsigned long long)prefix.header_size, (unsigned long long)(file_size - base));
    if (prefix.next_header_offset &&
        (base + prefix.next_header_offset + sizeof(HeaderPrefix) > file_size ||
         base + prefix.next_header_offset < base))
      return pfail(IREE_B200_STATUS_OUT_OF_RANGE,
                   "file buffer underrun verifying linked header at offset %llu (only %llu bytes available)",
                   (unsigned long long)prefix.next_header_offset, (unsigned long long)(file_size - base));
    if (prefix.version_major != 0)
      return pfail(IREE_B200_STATUS_UNIMPLEMENTED, "IRPA major version %u.%u not supported by this runtime",
                   prefix.version_major, prefix.version_minor);
    if (iree_b200_status_t st = parse_header_v0(file, file_size, base, prefix, index)) return st;
    if (!prefix.next_header_offset) break;
    base += prefix.next_header_offset;
  }
  return IREE_B200_STATUS_OK;
}

const Entry* find(const iree_b200_parameter_index_t* index, const char* key) {
  const size_t n = strlen(key);
  for (const Entry& e : index->entries)
    if (e.key.size() == n && memcmp(e.key.data(), key, n) == 0) return &e;
  return nullptr;
}

void export_entry(const Entry& e, iree_b200_parameter_entry_t* out) {
  memset(out, 0, sizeof *out);
  out->key = e.key.data();
  out->key_length = e.key.size();
  out->metadata = e.metadata.empty() ? nullptr : e.metadata.data();
  out->metadata_length = e.metadata.size();
  out->length = e.length;
  out->storage_type = e.type;
  out->file_offset = e.file_offset;
  out->pattern_length = e.pattern_length;
  memcpy(out->pattern, e.pattern, 16);
}

}  // namespace

extern "C" {

iree_b200_status_t iree_b200_parameter_index_parse(const void* data, size_t size,
                                                   iree_b200_parameter_index_t** out_index) {
  if (!out_index) return pfail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  *out_index = nullptr;
  if (!data && size) return pfail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  auto* index = new iree_b200_parameter_index_t();
  index->base = static_cast<const uint8_t*>(data);
  index->size = size;
  const iree_b200_status_t st = parse_archive(index->base, size, index);
  if (st) {
    delete index;
    return st;
  }
  *out_index = index;
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_b200_parameter_index_open(const char* path, iree_b200_parameter_index_t** out_index) {
  if (!path || !out_index) return pfail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  *out_index = nullptr;
  const int fd = open(path, O_RDONLY);
  if (fd < 0) return pfail(IREE_B200_STATUS_NOT_FOUND, "failed to open file '%s' (%s)", path, strerror(errno));
  struct stat sb;
  if (fstat(fd, &sb) != 0) {
    close(fd);
    return pfail(IREE_B200_STATUS_UNKNOWN, "fstat('%s') failed (%s)", path, strerror(errno));
  }
  void* map = nullptr;
  if (sb.st_size > 0) {
    map = mmap(nullptr, sb.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (map == MAP_FAILED) {
      close(fd);
      return pfail(IREE_B200_STATUS_UNKNOWN, "mmap('%s') failed (%s)", path, strerror(errno));
    }
  }
  iree_b200_parameter_index_t* index = nullptr;
  const iree_b200_status_t st = iree_b200_parameter_index_parse(map, static_cast<size_t>(sb.st_size), &index);
  if (st) {
    if (map) munmap(map, sb.st_size);
    close(fd);
    return st;
  }
  index->fd = fd;
  index->owns_mapping = true;
  *out_index = index;
  return IREE_B200_STATUS_OK;
}

void iree_b200_parameter_index_release(iree_b200_parameter_index_t* index) {
  if (!index) return;
  if (index->owns_mapping) {
    if (index->base) munmap(const_cast<uint8_t*>(index->base), index->size);
    if (index->fd >= 0) close(index->fd);
  }
  delete index;
}

int64_t iree_b200_parameter_index_count(const iree_b200_parameter_index_t* index) {
  return index ? static_cast<int64_t>(index->entries.size()) : 0;
}

iree_b200_status_t iree_b200_parameter_index_get(const iree_b200_parameter_index_t* index, int64_t i,
                                                 iree_b200_parameter_entry_t* out_entry) {
  if (!index || !out_entry) return pfail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  if (i < 0 || i >= static_cast<int64_t>(index->entries.size()))
    return pfail(IREE_B200_STATUS_OUT_OF_RANGE, "entry %lld out of range (have %zu)", (long long)i, index->entries.size());
  export_entry(index->entries[i], out_entry);
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_b200_parameter_index_lookup(const iree_b200_parameter_index_t* index, const char* key,
                                                    iree_b200_parameter_entry_t* out_entry) {
  if (!index || !key || !out_entry) return pfail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  const Entry* e = find(index, key);
  if (!e) return pfail(IREE_B200_STATUS_NOT_FOUND, "no parameter found in index with key '%s'", key);
  export_entry(*e, out_entry);
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_b200_parameter_read(const iree_b200_parameter_index_t* index, const char* key,
                                            uint64_t parameter_offset, void* host_ptr, uint64_t length) {
  if (!index || !key || (!host_ptr && length)) return pfail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  const Entry* e = find(index, key);
  if (!e) return pfail(IREE_B200_STATUS_NOT_FOUND, "no parameter found in index with key '%s'", key);
  if (parameter_offset > e->length || length > e->length - parameter_offset)
    return pfail(IREE_B200_STATUS_OUT_OF_RANGE, "parameter '%s' range [%llu, +%llu) exceeds its length %llu", key,
                 (unsigned long long)parameter_offset, (unsigned long long)length, (unsigned long long)e->length);
  uint8_t* dst = static_cast<uint8_t*>(host_ptr);
  if (e->type == IREE_B200_PARAMETER_STORAGE_FILE) {
    memcpy(dst, index->base + e->file_offset + parameter_offset, length);
  } else {
    const uint64_t pl = e->pattern_length ? e->pattern_length : 1;
    for (uint64_t i = 0; i < length; ++i) dst[i] = e->pattern[(parameter_offset + i) % pl];
  }
  return IREE_B200_STATUS_OK;
}

iree_b200_status_t iree_b200_parameter_load(iree_b200_context_t* context, const iree_b200_parameter_index_t* index,
                                            const char* key, uint64_t parameter_offset, void* device_ptr,
                                            uint64_t length) {
  if (!context || !index || !key || (!device_ptr && length)) return pfail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  const Entry* e = find(index, key);
  if (!e) return pfail(IREE_B200_STATUS_NOT_FOUND, "no parameter found in index with key '%s'", key);
  if (parameter_offset > e->length || length > e->length - parameter_offset)
    return pfail(IREE_B200_STATUS_OUT_OF_RANGE, "parameter '%s' range [%llu, +%llu) exceeds its length %llu", key,
                 (unsigned long long)parameter_offset, (unsigned long long)length, (unsigned long long)e->length);
  if (!length) return IREE_B200_STATUS_OK;
  iree_hal_b200_device_t* device = iree_b200_context_device(context);
  if (e->type == IREE_B200_PARAMETER_STORAGE_FILE) {
    // The source is the page-cache mapping of the archive: pageable, so the driver stages it.
    iree_b200_status_t st = iree_hal_b200_transfer_h2d(device, index->base + e->file_offset + parameter_offset, device_ptr,
                                                       length);
    if (!st) st = iree_hal_b200_device_synchronize(device);  // the mapping may go away after return
    return st;
  }
  // Splat: fill on the device. A one-byte pattern is a memset; longer patterns are expanded into
  // a host block holding a whole number of patterns, which is then copied as often as needed
  // (splats are load-time constants, so this is not on any hot path).
  const uint64_t pl = e->pattern_length ? e->pattern_length : 1;
  if (pl == 1) return iree_hal_b200_fill_buffer(device, device_ptr, length, e->pattern[0]);
  const uint64_t block_bytes = ((1u << 20) / pl) * pl;
  std::vector<uint8_t> block(block_bytes < length ? block_bytes : length);
  for (uint64_t i = 0; i < block.size(); ++i) block[i] = e->pattern[(parameter_offset + i) % pl];
  for (uint64_t done = 0; done < length; done += block.size()) {
    const uint64_t n = length - done < block.size() ? length - done : block.size();
    if (iree_b200_status_t st = iree_hal_b200_transfer_h2d(device, block.data(), static_cast<uint8_t*>(device_ptr) + done, n))
      return st;
  }
  return iree_hal_b200_device_synchronize(device);  // the block goes away on return
}

// Archive writer: same segment layout and alignment rules as the reference's builder
// (irpa_builder.c:46-100 sizes, :102-237 write): header, entry table (16-byte aligned entries,
// in the order given), metadata segment (names then metadata blobs, in entry order), storage
// segment aligned to the first data entry's alignment, file padded to 4096 bytes.
iree_b200_status_t iree_b200_parameter_archive_write(const char* path, int64_t entry_count,
                                                     const iree_b200_parameter_source_t* entries) {
  if (!path || (entry_count && !entries) || entry_count < 0) return pfail(IREE_B200_STATUS_INVALID_ARGUMENT, "NULL argument");
  uint64_t entry_segment_size = 0, metadata_size = 0, storage_size = 0, storage_alignment = 0;
  std::vector<uint64_t> storage_offsets(entry_count, 0);
  for (int64_t i = 0; i < entry_count; ++i) {
    const auto& s = entries[i];
    if (!s.key) return pfail(IREE_B200_STATUS_INVALID_ARGUMENT, "entry %lld has no key", (long long)i);
    if (s.storage_type == IREE_B200_PARAMETER_STORAGE_SPLAT) {
      if (s.pattern_length == 0 || s.pattern_length > 16 || (s.pattern_length & (s.pattern_length - 1)))
        return pfail(IREE_B200_STATUS_INVALID_ARGUMENT, "splat pattern length %u invalid; must be 1, 2, 4, 8, or 16 bytes",
                     s.pattern_length);
      entry_segment_size = align_up(entry_segment_size, kEntryAlignment) + sizeof(SplatEntry);
    } else if (s.storage_type == IREE_B200_PARAMETER_STORAGE_FILE) {
      const uint64_t alignment = s.alignment ? s.alignment : 64;
      storage_offsets[i] = align_up(storage_size, alignment);
      storage_size = storage_offsets[i] + s.length;
      if (!storage_alignment) storage_alignment = alignment;
      entry_segment_size = align_up(entry_segment_size, kEntryAlignment) + sizeof(DataEntry);
    } else {
      return pfail(IREE_B200_STATUS_INVALID_ARGUMENT, "unhandled entry type %d", s.storage_type);
    }
    metadata_size += strlen(s.key) + s.metadata_length;
  }
  HeaderV0 h;
  memset(&h, 0, sizeof h);
  h.prefix.magic = kMagic;
  h.prefix.header_size = sizeof h;
  h.entry_count = static_cast<uint64_t>(entry_count);
  h.entry_segment = {align_up(sizeof(HeaderV0), kEntryAlignment), entry_segment_size};
  h.metadata_segment = {h.entry_segment.offset + h.entry_segment.length, metadata_size};
  h.storage_segment = {align_up(h.metadata_segment.offset + h.metadata_segment.length, storage_alignment ? storage_alignment : 1),
                       storage_size};
  const uint64_t total = align_up(h.storage_segment.offset + storage_size, kFileAlignment);
  std::vector<uint8_t> image(total, 0);
  memcpy(image.data(), &h, sizeof h);
  uint64_t cursor = sizeof h, metadata_offset = 0;
  for (int64_t i = 0; i < entry_count; ++i) {
    const auto& s = entries[i];
    cursor = align_up(cursor, kEntryAlignment);
    EntryHeader eh;
    memset(&eh, 0, sizeof eh);
    eh.name = {metadata_offset, strlen(s.key)};
    metadata_offset += eh.name.length;
    eh.metadata = {s.metadata_length ? metadata_offset : 0, s.metadata_length};
    metadata_offset += s.metadata_length;
    if (s.storage_type == IREE_B200_PARAMETER_STORAGE_SPLAT) {
      SplatEntry e;
      memset(&e, 0, sizeof e);
      e.header = eh;
      e.header.entry_size = sizeof e;
      e.header.type = kEntrySplat;
      e.length = s.length;
      e.pattern_length = s.pattern_length;
      memcpy(e.pattern, s.pattern, s.pattern_length);
      memcpy(image.data() + cursor, &e, sizeof e);
      cursor += sizeof e;
    } else {
      DataEntry e;
      memset(&e, 0, sizeof e);
      e.header = eh;
      e.header.entry_size = sizeof e;
      e.header.type = kEntryData;
      e.header.minimum_alignment = 64;  // the builder records its default, whatever the caller asked for
      e.storage = {storage_offsets[i], s.length};
      memcpy(image.data() + cursor, &e, sizeof e);
      cursor += sizeof e;
      uint8_t* dst = image.data() + h.storage_segment.offset + storage_offsets[i];
      if (s.data) {
        memcpy(dst, s.data, s.length);
      } else if (s.pattern_length) {  // a data entry filled with a repeating pattern
        for (uint64_t b = 0; b < s.length; ++b) dst[b] = s.pattern[b % s.pattern_length];
      }
    }
  }
  uint64_t mcursor = h.metadata_segment.offset;
  for (int64_t i = 0; i < entry_count; ++i) {
    const auto& s = entries[i];
    memcpy(image.data() + mcursor, s.key, strlen(s.key));
    mcursor += strlen(s.key);
    if (s.metadata_length) memcpy(image.data() + mcursor, s.metadata, s.metadata_length);
    mcursor += s.metadata_length;
  }
  FILE* f = fopen(path, "wb");
  if (!f) return pfail(IREE_B200_STATUS_PERMISSION_DENIED, "failed to open '%s' for writing (%s)", path, strerror(errno));
  const size_t written = fwrite(image.data(), 1, image.size(), f);
  if (fclose(f) != 0 || written != image.size())
    return pfail(IREE_B200_STATUS_DATA_LOSS, "short write to '%s'", path);
  (void)kHeaderAlignment;
  return IREE_B200_STATUS_OK;
}

}  // extern "C"
