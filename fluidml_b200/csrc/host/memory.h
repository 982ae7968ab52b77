// Memory planning: lifetime records, the two planners and the resulting arena index.
// Same algorithms as the reference's structure/memory/ (info.cpp, linear.cpp, greedy.cpp,
// index.cpp), re-implemented on an ordered interval set, with an optional per-tenant
// alignment so every tensor base is valid for 16-byte vector access and TMA.
#pragma once
#include <cstddef>
#include <cstdint>
#include <deque>
#include <queue>
#include <string>
#include <tuple>
#include <unordered_map>
#include <vector>

namespace fluidml {
namespace memory {

// A tenant: lives from sequence index `start` to `end` (both inclusive), `size` bytes.
struct Info {
  std::string name;
  size_t start, end, size;
};

class Infos {
public:
  virtual ~Infos() = default;
  virtual bool IsEmpty() const = 0;
  virtual void Push(Info &&info) = 0;
  virtual Info Pop() = 0;
};

// FIFO (reference PlainInfos, info.cpp:20-34).
class PlainInfos : public Infos {
public:
  bool IsEmpty() const override { return infos_.empty(); }
  void Push(Info &&info) override { infos_.push_back(std::move(info)); }
  Info Pop() override { Info i = std::move(infos_.front()); infos_.pop_front(); return i; }

private:
  std::deque<Info> infos_;
};

// Largest first (reference GreedyInfos, info.cpp:36-52): a std::priority_queue ordered by
// size only, so ties come out in the same heap order as the reference's for the same
// sequence of pushes.
class GreedyInfos : public Infos {
public:
  struct Compare { bool operator()(const Info &l, const Info &r) const { return l.size < r.size; } };
  bool IsEmpty() const override { return infos_.empty(); }
  void Push(Info &&info) override { infos_.push(std::move(info)); }
  Info Pop() override { Info i = infos_.top(); infos_.pop(); return i; }

private:
  std::priority_queue<Info, std::vector<Info>, Compare> infos_;
};

class Index {
public:
  void Set(const std::string &name, size_t offset, size_t size) { map_.insert({name, {offset, size}}); }
  bool Has(const std::string &name) const { return map_.count(name) != 0; }
  size_t Get(const std::string &name) const { return map_.at(name).first; }
  size_t GetSize(const std::string &name) const { return map_.at(name).second; }
  size_t GetMaximum() const;  // arena bytes = max(offset + size), index.cpp:17-24
  const std::unordered_map<std::string, std::pair<size_t, size_t>> &All() const { return map_; }

private:
  std::unordered_map<std::string, std::pair<size_t, size_t>> map_;
};

class Plan {
public:
  virtual ~Plan() = default;
  virtual Index Run(Infos &infos) const = 0;
};

// Bump allocation in pop order (linear.cpp:5-15).
class LinearPlan : public Plan {
public:
  explicit LinearPlan(size_t alignment = 1) : alignment_(alignment) {}
  Index Run(Infos &infos) const override;

private:
  size_t alignment_;
};

// greedy.cpp:239-270: pop largest first; byte ranges of already placed tenants whose
// lifetime [start, end+1] intersects (inclusive test, greedy.cpp:61-69) are busy; take the
// smallest gap BETWEEN two busy ranges that fits, else append after the last busy range;
// the gap in front of the first busy range is never used (greedy.cpp:180-207).
class GreedyPlan : public Plan {
public:
  explicit GreedyPlan(size_t alignment = 1) : alignment_(alignment) {}
  Index Run(Infos &infos) const override;

private:
  size_t alignment_;
};

}  // namespace memory
}  // namespace fluidml
