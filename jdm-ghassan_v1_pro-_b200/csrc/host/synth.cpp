#include "synth.hpp"

#include <algorithm>
#include <cmath>
#include <cstdio>

#include "dataset.hpp"
#include "unicode.hpp"

namespace gbh {

namespace {

template <typename T>
const T& pick(Rng& rng, const std::vector<T>& v) {
  return v[static_cast<size_t>(rng.below(v.size()))];
}

u64 hash_str(const std::string& s, u64 h = 0xcbf29ce484222325ULL) {
  for (unsigned char c : s) {
    h ^= c;
    h *= 0x100000001b3ULL;
  }
  return h;
}

std::string replace_all(std::string s, const std::string& what, const std::string& with) {
  for (size_t p = s.find(what); p != std::string::npos; p = s.find(what, p + with.size())) s.replace(p, what.size(), with);
  return s;
}

bool contains(const std::string& s, const char* needle) { return s.find(needle) != std::string::npos; }

std::string lower_ascii(std::string s) {
  for (auto& c : s)
    if (c >= 'A' && c <= 'Z') c = static_cast<char>(c - 'A' + 'a');
  return s;
}

bool is_arabic_letter(u32 cp) { return (cp >= 0x0621 && cp <= 0x064A) || cp == 0x06AF || cp == 0x06A4 || cp == 0x067E || cp == 0x06A9; }
bool is_diacritic(u32 cp) { return (cp >= 0x064B && cp <= 0x0652) || cp == 0x0670 || cp == 0x0640; }

}  // namespace

// ================================================================================================ transliteration
std::string arabic_to_arabizi(const std::string& arabic, Rng& rng, bool heavy_digits) {
  const std::vector<u32> cps = uni::to_cps(arabic);
  std::string out;
  out.reserve(arabic.size());
  auto letter_at = [&](size_t i) { return i < cps.size() && is_arabic_letter(cps[i]); };
  for (size_t i = 0; i < cps.size(); ++i) {
    const u32 c = cps[i];
    if (is_diacritic(c)) {
      if (c == 0x0651 && !out.empty() && std::isalpha(static_cast<unsigned char>(out.back()))) out.push_back(out.back());  // shadda doubles
      continue;
    }
    const bool word_start = i == 0 || !letter_at(i - 1);
    const bool word_end = !letter_at(i + 1);
    // definite article: "ال" at a word start is spoken "l" (or "el"); before a sun letter the l is swallowed
    if (word_start && c == 0x0627 && i + 2 < cps.size() && cps[i + 1] == 0x0644 && letter_at(i + 2)) {
      out += rng.uniform() < 0.75 ? "l" : "el";
      ++i;
      continue;
    }
    switch (c) {
      case 0x0627: out += word_start ? "a" : (rng.uniform() < 0.85 ? "a" : "e"); break;          // ا
      case 0x0623: case 0x0622: out += "a"; break;                                                // أ آ
      case 0x0625: out += "i"; break;                                                             // إ
      case 0x0628: out += "b"; break;
      case 0x062A: case 0x0637: out += "t"; break;                                                // ت ط
      case 0x062B: out += "t"; break;
      case 0x062C: out += "j"; break;
      case 0x062D: out += heavy_digits || rng.uniform() < 0.5 ? "7" : "h"; break;                  // ح
      case 0x062E: out += !heavy_digits && rng.uniform() < 0.2 ? "5" : "kh"; break;                // خ
      case 0x062F: case 0x0630: case 0x0636: case 0x0638: out += "d"; break;                      // د ذ ض ظ
      case 0x0631: out += "r"; break;
      case 0x0632: out += "z"; break;
      case 0x0633: case 0x0635: out += "s"; break;
      case 0x0634: out += rng.uniform() < 0.8 ? "ch" : "sh"; break;                                // ش
      case 0x0639: out += heavy_digits || rng.uniform() < 0.6 ? "3" : "a"; break;                  // ع
      case 0x063A: out += "gh"; break;
      case 0x0641: out += "f"; break;
      case 0x0642: out += heavy_digits || rng.uniform() < 0.5 ? "9" : (rng.uniform() < 0.5 ? "q" : "k"); break;   // ق
      case 0x0643: case 0x06A9: out += "k"; break;
      case 0x0644: out += "l"; break;
      case 0x0645: out += "m"; break;
      case 0x0646: out += "n"; break;
      case 0x0647: out += word_end ? (rng.uniform() < 0.5 ? "h" : "") : "h"; break;                // ه
      case 0x0629: out += "a"; break;                                                             // ة
      case 0x0648:                                                                                // و
        if (word_start) out += "w";
        else if (word_end) out += rng.uniform() < 0.6 ? "ou" : "o";
        else out += rng.uniform() < 0.5 ? "o" : "ou";
        break;
      case 0x064A: out += word_start ? "y" : "i"; break;                                          // ي
      case 0x0649: out += "a"; break;                                                             // ى
      case 0x0621: case 0x0626: case 0x0624: out += heavy_digits ? "2" : "'"; break;               // ء ئ ؤ
      case 0x06AF: out += "g"; break;
      case 0x06A4: out += "v"; break;
      case 0x067E: out += "p"; break;
      case 0x061F: out += "?"; break;
      case 0x060C: out += ","; break;
      case 0x061B: out += ";"; break;
      default:
        if (c < 0x80) out.push_back(static_cast<char>(c));
        else if (c >= 0x0660 && c <= 0x0669) out.push_back(static_cast<char>('0' + (c - 0x0660)));
        else if (c < 0x0600 || c > 0x06FF) uni::encode(c, out);   // keep emoji, Latin-1, ...
        break;
    }
  }
  return out;
}

std::string orthographic_noise(const std::string& latin, Rng& rng, double rate) {
  std::string out;
  out.reserve(latin.size() + 8);
  for (size_t i = 0; i < latin.size(); ++i) {
    const char c = latin[i];
    const double r = rng.uniform();
    const bool inner = i > 0 && i + 1 < latin.size() && std::isalpha(static_cast<unsigned char>(latin[i - 1])) &&
                       std::isalpha(static_cast<unsigned char>(latin[i + 1]));
    if ((c == 'a' || c == 'e' || c == 'i' || c == 'o') && inner && r < rate) continue;           // dropped short vowel
    if (c == 'o' && i + 1 < latin.size() && latin[i + 1] == 'u' && r < rate * 4) { out += "o"; ++i; continue; }
    if (c == 'c' && i + 1 < latin.size() && latin[i + 1] == 'h' && r < rate * 2) { out += "sh"; ++i; continue; }
    if (c == '9' && r < rate * 2) { out += "q"; continue; }
    if (c == ' ' && r < rate * 0.3) continue;                                                     // lost space
    out.push_back(c);
    if (std::isalpha(static_cast<unsigned char>(c)) && r > 1.0 - rate * 0.5) out.push_back(c);  // doubled letter
  }
  return out;
}

double char_entropy_bits(const std::string& text) {
  std::unordered_map<u32, u64> freq;
  u64 n = 0;
  for (size_t i = 0; i < text.size();) {
    ++freq[uni::decode(text, i)];
    ++n;
  }
  if (n == 0) return 0.0;
  double h = 0.0;
  for (const auto& kv : freq) {
    const double p = static_cast<double>(kv.second) / static_cast<double>(n);
    h -= p * std::log2(p);
  }
  return h;
}

double distinct_word_ratio(const std::string& text) {
  std::unordered_set<std::string> seen;
  u64 n = 0;
  std::string w;
  auto flush = [&]() {
    if (!w.empty()) {
      seen.insert(w);
      ++n;
      w.clear();
    }
  };
  for (char c : text) {
    if (c == ' ' || c == '\n' || c == '\t') flush();
    else w.push_back(c);
  }
  flush();
  return n == 0 ? 0.0 : static_cast<double>(seen.size()) / static_cast<double>(n);
}

std::string SynthStats::summary() const {
  // plain string building: stream insertion of integers goes through locale facets, which crashed here once another
  // extension module with its own copy of the C++ runtime (pyarrow) had been loaded into the process first
  auto num = [](u64 v) { return std::to_string(static_cast<unsigned long long>(v)); };
  std::string s = "accepted " + num(accepted) + " of " + num(attempts) + " attempts (duplicate " + num(rejected_duplicate) +
                  ", template cap " + num(rejected_template_cap) + ", style " + num(rejected_style) + ", entropy " +
                  num(rejected_entropy) + "); scripts";
  for (const auto& kv : by_script) s += " " + kv.first + "=" + num(kv.second);
  s += "; domains";
  for (const auto& kv : by_domain) s += " " + kv.first + "=" + num(kv.second);
  return s;
}

// ================================================================================================ Darija content
namespace {

struct Pair {
  const char* user;
  const char* assistant;
};
struct Domain {
  const char* name;
  std::vector<Pair> pairs;
};

// Slot values, Arabic script.  {city} {dish} {item} {skill} {day} {sport} {device} {sym} {price} {n} are filled below.
const std::vector<std::string> CITIES = {"الرباط", "كازا", "مراكش", "فاس", "طنجة", "أكادير", "وجدة", "تطوان", "مكناس", "الصويرة"};
const std::vector<std::string> DISHES = {"الطاجين", "الكسكس", "الحريرة", "البسطيلة", "الرفيسة", "الزعلوك", "البيصارة", "المسمن"};
const std::vector<std::string> ITEMS = {"تيليفون", "سباط", "جاكيطة", "حاسوب", "ساعة", "شكارة", "طابلة", "كتاب"};
const std::vector<std::string> SKILLS = {"البرمجة", "الإنجليزية", "الطبخ", "السياقة", "الرياضيات", "التصوير", "الخياطة", "المحاسبة"};
const std::vector<std::string> DAYS = {"الاثنين", "الثلاثاء", "الأربعاء", "الخميس", "الجمعة", "السبت", "الأحد"};
const std::vector<std::string> SPORTS = {"الكورة", "الجري", "السباحة", "الباسكيط", "التنس"};
const std::vector<std::string> DEVICES = {"التيليفون", "البيسي", "الراوتر", "الطابليت", "التلفازة"};
const std::vector<std::string> SYMPTOMS = {"الراس كيضرني", "عندي السخانة", "كرشي كتوجعني", "ما كنعسش مزيان", "عندي الكحة"};

const std::vector<Domain> DOMAINS = {
    {"greetings",
     {{"السلام عليكم، كيداير؟", "وعليكم السلام، لاباس الحمد لله. ونتا كيداير مع الوقت؟"},
      {"صباح الخير، كيف صبحتي؟", "صباح النور، بخير الحمد لله. شنو غادي دير اليوم؟"},
      {"أهلا، شحال هادي ما شفناك", "أهلا بيك، بصح توحشناك. كيف دايرة معاك الخدمة والصحة؟"},
      {"مسا الخير", "مسا النور، كيف داز نهارك؟"},
      {"واش كلشي بخير عندك؟", "كلشي مزيان الحمد لله، غير شوية ديال العيا. ونتا؟"}}},
    {"daily_life",
     {{"شنو ندير نهار {day}؟ ما عندي حتى برنامج", "إلا كان الجو زوين خرج تمشى ولا تلاقى مع صحابك، وإلا بقى فالدار رتب حوايجك وقرا شي حاجة."},
      {"كيفاش ننظم وقتي؟ ديما كنتعطل", "كتب فالليل ثلاثة ديال الحوايج المهمين ديال غدا، وبدا بالصعيبة فالصباح ملي كتكون باقي نشيط."},
      {"بغيت نبدل الدار، منين نبدا؟", "حدد الميزانية أولا، من بعد شوف الأحياء القريبة من الخدمة، وسول الجيران قبل ما تكري."},
      {"الجيران كيديرو الصداع بالليل", "هضر معاهم بالتي هي أحسن أولا، غالبا ما عارفينش. إلا ما تبدل والو سول السانديك."}}},
    {"food",
     {{"كيفاش كنديرو {dish}؟", "خاصك المقادير ديال {dish} طريين، طيب على نار هادية وما تزربش، والسر كامل فالتوابل والصبر."},
      {"شنو نطيب للعشا اليوم؟ عندي غير شوية ديال الخضرة", "دير شي {dish} خفيف ولا شلاضة مع البيض، ساهلة وكتشبع."},
      {"فين نلقى {dish} مزيان ف {city}؟", "ف {city} سول على المطاعم الشعبية قرب المدينة القديمة، تما كيطيبو {dish} بحال ديال الدار."},
      {"بغيت ننقص من السكر، شنو ندير؟", "نقص شوية بشوية: أتاي بلا سكر بزاف، وبدل الحلوى بالفاكية، وقرا المكونات قبل ما تشري."}}},
    {"shopping",
     {{"بشحال هاد {item}؟", "هاد {item} كيدير {price} درهم، ولكن إلا خديتي جوج نقص ليك شوية."},
      {"بغيت نشري {item} ولكن ما عارفش واش نستنى التخفيضات", "إلا ما كنتيش مزروب استنى، التخفيضات غالبا كيكونو فآخر الموسم. قارن الأثمنة ف جوج ولا ثلاثة ديال البلايص."},
      {"واش {price} درهم ثمن معقول ل {item}؟", "على حساب الجودة، ولكن {price} درهم ل {item} ثمن متوسط. شوف واش فيه الضمانة."},
      {"شريت {item} وطلع خاسر، شنو ندير؟", "رجع عند البائع بالتوصيل، من حقك يبدلو ليك ولا يرجع ليك فلوسك إلا مازال فالأجل."}}},
    {"travel",
     {{"كيفاش نمشي من {city} ل {city2}؟", "من {city} ل {city2} كاين التران والكار. التران مريح كثر، والكار أرخص شوية."},
      {"شنو نزور ف {city}؟", "ف {city} ما تفوتش المدينة القديمة والأسواق، وإلا عندك الوقت دوز للبحر ولا الجبل القريب."},
      {"بغيت نسافر نهار {day}، واش نحجز من دابا؟", "أحسن تحجز من دابا، نهار {day} كيكون الزحام والأثمنة كيطلعو ملي كيقرب الوقت."},
      {"شحال ديال الوقت خاصني ف {city}؟", "جوج أيام ولا ثلاثة كافيين باش تشوف أهم البلايص ف {city} بلا زربة."}}},
    {"health",
     {{"{sym} من البارح، شنو ندير؟", "ارتاح وشرب الما بزاف. إلا بقى الحال هكا أكثر من يومين ولا زاد عليك، خاصك تشوف طبيب، أنا ما نقدرش نعوضو."},
      {"كيفاش نبدا الرياضة وأنا عمري ما درتها؟", "بدا بالمشي نص ساعة فالنهار، ومن بعد زيد شوية بشوية. المهم هو الاستمرار ماشي الشدة."},
      {"ما كنعسش مزيان هاد الأيام", "نقص من القهوة والتيليفون قبل النعاس، ونعس وفيق فنفس الوقت كل نهار. إلا طول المشكل سول طبيب."},
      {"شنو ناكل باش نبقى بصحتي؟", "كثر من الخضرة والفاكية والقطاني، ونقص من المقليات والسكر، وشرب الما كافي."}}},
    {"study",
     {{"بغيت نتعلم {skill}، منين نبدا؟", "بدا بالأساسيات ديال {skill} من مصدر واحد مزيان، وطبق كل نهار شوية. المشاريع الصغار كيعلمو كثر من القراية بوحدها."},
      {"عندي امتحان نهار {day} وما قريت والو", "قسم الدروس على الأيام اللي بقات، بدا بالمهم، ودير تمارين ديال السنوات اللي فاتو. ونعس مزيان ليلة الامتحان."},
      {"كنسى بزاف داكشي اللي كنقرا", "راجع داكشي من بعد نهار، ومن بعد سيمانة. وشرح الدرس لشي واحد آخر، هادي أحسن طريقة باش يثبت."},
      {"واش نقرا بوحدي ولا مع صحابي؟", "بجوج مزيانين: بوحدك باش تفهم، ومع صحابك باش تراجع وتشوف فين ناقص."}}},
    {"work",
     {{"كنقلب على خدمة ف {skill}، شنو ندير؟", "وجد سيفي قصير وواضح، ودير شي مشاريع كيبينو شنو كتعرف ف {skill}، وصيفط لبزاف ديال الشركات ماشي غير وحدة."},
      {"عندي مقابلة ديال الخدمة نهار {day}", "قرا على الشركة، ووجد أمثلة من التجربة ديالك، وسول حتى نتا فالآخر. ووصل قبل الوقت."},
      {"المدير ديالي ما كيقدرش الخدمة ديالي", "طلب منو لقاء قصير وسولو شنو كيتسنى منك بالضبط، وكتب الإنجازات ديالك باش تبينهم بالأرقام."},
      {"واش نبدل الخدمة ولا نبقى؟", "كتب شنو كيعجبك وشنو لا فالخدمة ديال دابا، وقارن مع العرض الجديد: الصالير، التعلم، والراحة. القرار ديالك فالآخر."}}},
    {"tech",
     {{"{device} ديالي ولا ثقيل بزاف", "مسح التطبيقات اللي ما كتخدمش بيهم، وخوي شوية من الذاكرة، وعاود شعلو. إلا بقى ثقيل شوف واش كاين تحديث."},
      {"كيفاش نحمي الحساب ديالي من السرقة؟", "دير كلمة سر طويلة ومختلفة لكل حساب، وفعل التحقق بجوج مراحل، وما تفتحش الروابط اللي ما عارفش منين جاو."},
      {"{device} ما بغاش يتكونيكطا بالويفي", "طفي الويفي وعاود شعلو، ونسى الشبكة وعاود دخل كلمة السر. إلا ما خدمش عاود شعل الراوتر."},
      {"شنو الفرق بين الرام والتخزين؟", "الرام هي الذاكرة اللي كيخدم بيها الجهاز دابا وكتخوى ملي كيطفى، والتخزين هو فين كيبقاو الملفات ديالك ديما."}}},
    {"family",
     {{"ولدي ما بغاش يقرا", "حاول تفهم علاش: واش الدرس صعيب ولا شي حاجة فالمدرسة؟ دير ليه وقت محدد للقراية وشجعو على المجهود ماشي غير النقطة."},
      {"بغيت ندير مفاجأة لمي", "وجد ليها شي حاجة كتبغيها: غدا فالدار مع العائلة ولا هدية بسيطة مع كلمة زوينة. الحضور ديالك هو أهم حاجة."},
      {"تخاصمت مع خويا", "خلي الأعصاب يبردو أولا، ومن بعد هضر معاه بهدوء وسمع ليه. غالبا المشكل كيكون سوء تفاهم صغير."}}},
    {"weather",
     {{"كيف داير الجو ف {city}؟", "ما عنديش معلومات حية على الجو، ولكن ف {city} فهاد الوقت من العام غالبا كيكون معتدل. شوف تطبيق الطقس باش تتأكد."},
      {"واش نخرج بلا جاكيطة اليوم؟", "ما نقدرش نشوف الجو ديال دابا، ولكن دي معاك شي حاجة خفيفة، الصباح والليل كيبردو."}}},
    {"sports",
     {{"بغيت نبدا {sport}، شنو خاصني؟", "باش تبدا {sport} خاصك غير حوايج مريحين والصبر. بدا بجوج مرات فالسيمانة وزيد من بعد."},
      {"شكون ربح الماتش البارح؟", "ما عنديش النتائج ديال البارح، أنا ما كنتبعش الأخبار الحية. شوف شي موقع رياضي باش تعرف."},
      {"كيفاش نحسن اللياقة ديالي ف {sport}؟", "نوع التمارين: نهار للسرعة، نهار للقوة، ونهار للراحة. وكول مزيان ونعس كافي."}}},
    {"money",
     {{"كيفاش نجمع الفلوس؟ الصالير كيسالي قبل آخر الشهر", "كتب المصاريف ديالك شهر كامل باش تعرف فين كيمشيو، وحط عشرة فالمية على جنب أول ما تخلص."},
      {"واش ناخد كريدي باش نشري {item}؟", "إلا {item} ماشي ضروري دابا، أحسن تجمع ليه. الكريدي كيزيد عليك الفوائد وكيربطك شهور."},
      {"بغيت نبدا مشروع صغير", "بدا بفكرة بسيطة وجربها بأقل مصاريف، وسول الناس واش غادي يشريو قبل ما تحط فلوسك كاملين."}}},
};

const std::vector<Pair> FOLLOWUPS = {
    {"وشنو آخر؟", "كاين حتى هادي: خود وقتك وما تزربش، وكل مرة زيد شوية على اللي درتي قبل."},
    {"عطيني مثال", "مثلا: بدا اليوم بحاجة صغيرة كتاخد ربع ساعة، وغدا زيد عليها شوية، وهكا حتى تولي عادة."},
    {"وعلاش؟", "حيت الطريقة اللي كتبدا بشوية وكتكمل هي اللي كتبقى، أما اللي كيبدا بالزربة غالبا كيحبس دغيا."},
    {"شحال ديال الوقت خاصني؟", "على حسابك، ولكن غالبا شي سيمانات قليلة باش تبدا تشوف الفرق إلا كنتي مواظب."},
    {"واخا، وإلا ما خدمش هادشي؟", "إلا ما خدمش جرب طريقة أخرى ولا سول شي واحد عندو التجربة، ماشي مشكل تبدل الخطة."},
    {"شكرا بزاف", "العفو، مرحبا بيك فأي وقت. إلا احتاجيتي شي حاجة أخرى أنا هنا."},
};
const std::vector<Pair> CORRECTIONS = {
    {"لا، ماشي هادشي اللي قصدت", "سمح ليا، فهمتك غلط. عاود ليا شنو بغيتي بالضبط ونجاوبك على قد السؤال."},
    {"غلطتي، أنا سولتك على حاجة أخرى", "عندك الحق، سمح ليا. وضح ليا السؤال مرة أخرى باش نعطيك الجواب الصحيح."},
    {"هاد الجواب طويل بزاف، لخص ليا", "واخا، باختصار: بدا بالمهم، دير خطوة وحدة فالنهار، وراجع فآخر السيمانة."},
};
const std::vector<Pair> CLARIFY = {
    {"هاداك", "ما فهمتش مزيان، واش تقدر توضح ليا على شنو كتهضر؟"},
    {"دير ليا داكشي", "شنو بالضبط بغيتي ندير؟ عطيني شوية ديال التفاصيل باش نعاونك."},
    {"كيفاش؟", "على شنو كتسول بالضبط؟ عاود ليا السؤال كامل باش نجاوبك مزيان."},
};
// the assistant says where its limits are, politely, and offers something it can do
const std::vector<Pair> GOVERNOR = {
    {"عطيني دوا نشربو بلا ما نمشي للطبيب", "ما نقدرش نوصف ليك دوا، هادي خدمة الطبيب ولا الفرمسيان. اللي نقدر نقول ليك هو ترتاح وتشرب الما وتمشي تشوف مختص إلا طول الحال."},
    {"قول ليا شكون غادي يربح الانتخابات", "ما نقدرش نتنبأ بهادشي وما عنديش رأي سياسي. نقدر نشرح ليك كيفاش كتخدم الانتخابات إلا بغيتي."},
    {"كتب ليا رسالة نسب فيها جاري", "ما غاديش نعاونك تسب شي واحد. إلا بغيتي نعاونك تكتب ليه رسالة محترمة كتشرح فيها المشكل، مرحبا."},
    {"واش متأكد مية فالمية؟", "لا، ما نقدرش نكون متأكد مية فالمية، نقدر نغلط. أحسن تتأكد من مصدر رسمي فالحوايج المهمين."},
};
const std::vector<Pair> MSA = {
    {"كيف حالك اليوم؟", "أنا بخير، شكراً لك. كيف يمكنني مساعدتك اليوم؟"},
    {"ما هي عاصمة المغرب؟", "عاصمة المغرب هي مدينة الرباط، وتقع على ساحل المحيط الأطلسي."},
    {"هل يمكنك أن تشرح لي هذا الموضوع؟", "بكل سرور، سأشرح لك الموضوع خطوة بخطوة، وأخبرني إن بقي شيء غير واضح."},
    {"أريد أن أتعلم لغة جديدة", "فكرة جيدة. ابدأ بالكلمات الأكثر استعمالاً، واستمع يومياً ولو لربع ساعة، وتحدث دون خوف من الخطأ."},
    {"ما الفرق بين الطقس والمناخ؟", "الطقس هو حالة الجو في وقت قصير ومكان محدد، أما المناخ فهو معدل حالة الجو على مدى سنوات طويلة."},
};
const std::vector<std::string> FRENCH = {"s'il te plaît", "merci", "d'accord", "normalement", "en fait", "bon", "voilà", "c'est bon"};
const std::vector<std::string> SYSTEMS_AR = {"نتا مساعد مغربي كتهضر بالدارجة بطريقة طبيعية ومختصرة.",
                                             "جاوب بالدارجة المغربية، بلا تطويل، وقول الصراحة ملي ما تعرفش."};
const std::vector<std::string> SYSTEMS_LATN = {"nta mosa3id maghribi, jaweb b darija b tariqa 9sira w wad7a.",
                                               "jaweb b darija maghribiya, bla tatwil, w 9oul ma3reftch mli ma t3rafch."};
const std::vector<std::string> SYSTEMS_MSA = {"أنت مساعد يجيب باللغة العربية الفصحى بإيجاز ووضوح."};

// One set of slot values per exchange: the question and its answer must name the same city, dish, price...
struct SlotPicks {
  std::map<std::string, std::string> chosen;
  u64 hash = 0;
};

std::string fill_slots(std::string t, Rng& rng, SlotPicks& picks) {
  auto sub = [&](const char* key, const std::vector<std::string>& values) {
    if (t.find(key) == std::string::npos) return;
    auto it = picks.chosen.find(key);
    if (it == picks.chosen.end()) {
      const size_t i = static_cast<size_t>(rng.below(values.size()));
      picks.hash = picks.hash * 1315423911ULL + i + 1;
      it = picks.chosen.emplace(key, values[i]).first;
    }
    t = replace_all(t, key, it->second);
  };
  sub("{city2}", CITIES);
  sub("{city}", CITIES);
  sub("{dish}", DISHES);
  sub("{item}", ITEMS);
  sub("{skill}", SKILLS);
  sub("{day}", DAYS);
  sub("{sport}", SPORTS);
  sub("{device}", DEVICES);
  sub("{sym}", SYMPTOMS);
  if (t.find("{price}") != std::string::npos) {
    auto it = picks.chosen.find("{price}");
    if (it == picks.chosen.end())
      it = picks.chosen.emplace("{price}", std::to_string(50 * (1 + static_cast<int>(rng.below(60))))).first;
    t = replace_all(t, "{price}", it->second);
  }
  return t;
}

// a small word problem with its worked answer (the numbers are drawn, the arithmetic is done here)
void reasoning_turn(Rng& rng, std::string& user, std::string& assistant) {
  const int kind = static_cast<int>(rng.below(3));
  char buf[512];
  if (kind == 0) {
    const int n = 2 + static_cast<int>(rng.below(8)), p = 5 * (1 + static_cast<int>(rng.below(30))), paid = ((n * p) / 100 + 1) * 100;
    std::snprintf(buf, sizeof buf, "شريت %d ديال الحوايج، كل وحدة ب %d درهم، وعطيت %d درهم. شحال خاصو يرد ليا؟", n, p, paid);
    user = buf;
    std::snprintf(buf, sizeof buf, "%d ضرب %d كتعطي %d درهم. عطيتي %d، يعني خاصو يرد ليك %d درهم.", n, p, n * p, paid, paid - n * p);
    assistant = buf;
  } else if (kind == 1) {
    const int km = 20 * (2 + static_cast<int>(rng.below(20))), speed = 20 * (2 + static_cast<int>(rng.below(5)));
    const int h = km / speed, m = (km % speed) * 60 / speed;
    std::snprintf(buf, sizeof buf, "الطريق فيها %d كيلومتر وأنا غادي ب %d كيلومتر فالساعة. شحال ديال الوقت غادي نبقى؟", km, speed);
    user = buf;
    std::snprintf(buf, sizeof buf, "قسم %d على %d: غادي تبقى تقريبا %d ساعة و %d دقيقة، بلا ما نحسبو الوقفات.", km, speed, h, m);
    assistant = buf;
  } else {
    const int total = 100 * (5 + static_cast<int>(rng.below(40))), pct = 5 * (1 + static_cast<int>(rng.below(8)));
    std::snprintf(buf, sizeof buf, "الثمن هو %d درهم وكاين تخفيض ديال %d فالمية. شحال غادي نخلص؟", total, pct);
    user = buf;
    std::snprintf(buf, sizeof buf, "%d فالمية من %d هي %d درهم، إذن غادي تخلص %d درهم.", pct, total, total * pct / 100, total - total * pct / 100);
    assistant = buf;
  }
}

}  // namespace

std::vector<std::string> DarijaSynth::domains() {
  std::vector<std::string> v;
  for (const auto& d : DOMAINS) v.emplace_back(d.name);
  return v;
}

DarijaSynth::DarijaSynth(const SynthConfig& cfg) : cfg_(cfg), rng_(cfg.seed) {}

bool DarijaSynth::build(SynthConversation& c) {
  Rng& r = rng_;
  const double tot = std::max(1e-9, cfg_.p_arabic_script + cfg_.p_latin_script + cfg_.p_msa);
  const double u = r.uniform() * tot;
  c.script = u < cfg_.p_arabic_script ? "arab" : (u < cfg_.p_arabic_script + cfg_.p_latin_script ? "latn" : "msa");
  const int span = std::max(0, cfg_.max_turns - cfg_.min_turns);
  const int n_msgs = cfg_.min_turns + static_cast<int>(r.below(static_cast<u64>(span) + 1));
  const int exchanges = std::max(1, (n_msgs + 1) / 2);
  const bool heavy = r.uniform() < cfg_.p_heavy_digits;
  const Domain& dom = pick(r, DOMAINS);
  c.domain = c.script == "msa" ? "msa" : dom.name;
  c.messages.clear();
  u64 tid = hash_str(c.domain);
  std::vector<u64> in_conv;
  for (int e = 0; e < exchanges; ++e) {
    std::string q, a;
    SlotPicks picks;
    const double x = r.uniform();
    const bool later = e > 0;
    int which = -1;
    const std::vector<Pair>* table = nullptr;
    double acc = 0.0;
    if (c.script == "msa") table = &MSA;
    else if (later && x < (acc += cfg_.p_correction)) table = &CORRECTIONS;
    else if (later && x < (acc += cfg_.p_misunderstand)) table = &CLARIFY;
    else if (later && x < (acc += cfg_.p_governor)) table = &GOVERNOR;
    else if (later && x < (acc += cfg_.p_reasoning)) { reasoning_turn(r, q, a); tid = tid * 31 + 7; }
    else if (later && x < (acc += cfg_.p_followup)) table = &FOLLOWUPS;
    else table = &dom.pairs;
    if (table != nullptr) {
      // a conversation does not ask the same thing twice: redraw a few times when the template was already used in it
      for (int tries = 0; tries < 4; ++tries) {
        which = static_cast<int>(r.below(table->size()));
        const u64 h = hash_str((*table)[static_cast<size_t>(which)].user);
        if (std::find(in_conv.begin(), in_conv.end(), h) == in_conv.end()) {
          in_conv.push_back(h);
          break;
        }
      }
      q = fill_slots((*table)[static_cast<size_t>(which)].user, r, picks);
      a = fill_slots((*table)[static_cast<size_t>(which)].assistant, r, picks);
      tid = tid * 1099511628211ULL + hash_str((*table)[static_cast<size_t>(which)].user);
      if (e == 0) {
        int& used = uses_[tid];
        if (used >= cfg_.max_template_uses) {
          ++stats_.rejected_template_cap;
          return false;
        }
        ++used;
      }
    }
    if (c.script != "msa" && r.uniform() < cfg_.p_french_switch) q += " " + pick(r, FRENCH);
    if (c.script == "latn") {
      q = orthographic_noise(arabic_to_arabizi(q, r, heavy), r, cfg_.noise_rate);
      a = arabic_to_arabizi(a, r, heavy);
    }
    c.messages.push_back({"user", q});
    c.messages.push_back({"assistant", a});
  }
  if (cfg_.include_system && r.uniform() < cfg_.p_system) {
    const auto& sys = c.script == "latn" ? SYSTEMS_LATN : (c.script == "msa" ? SYSTEMS_MSA : SYSTEMS_AR);
    c.messages.insert(c.messages.begin(), SynthMessage{"system", pick(r, sys)});
  }
  c.template_id = tid;
  return true;
}

bool DarijaSynth::generate(SynthConversation& out) {
  ++stats_.attempts;
  SynthConversation c;
  if (!build(c)) return false;
  std::string all;
  for (const auto& m : c.messages)
    if (m.role != "system") all += m.content + "\n";
  const u64 key = hash_str(all);
  if (!seen_.insert(key).second) {
    ++stats_.rejected_duplicate;
    return false;
  }
  // style: no assistant turn may read like boilerplate, and the script must be what was drawn
  for (size_t i = 0; i + 1 < c.messages.size(); ++i) {
    if (c.messages[i].role != "user" || c.messages[i + 1].role != "assistant") continue;
    if (has_hard_ai_boilerplate(c.messages[i + 1].content)) {
      ++stats_.rejected_style;
      return false;
    }
  }
  const LangScore ls = classify_language(all);
  const bool script_ok = c.script == "latn" ? ls.latin_ratio > ls.arabic_ratio : ls.arabic_ratio >= ls.latin_ratio;
  if (!script_ok) {
    ++stats_.rejected_style;
    return false;
  }
  if (char_entropy_bits(all) < cfg_.min_entropy_bits || distinct_word_ratio(all) < cfg_.min_distinct_words) {
    ++stats_.rejected_entropy;
    return false;
  }
  ++stats_.accepted;
  ++stats_.by_domain[c.domain];
  ++stats_.by_script[c.script];
  out = std::move(c);
  return true;
}

std::vector<SynthConversation> DarijaSynth::generate_many(int n) {
  std::vector<SynthConversation> out;
  const u64 budget = static_cast<u64>(std::max(1, n)) * static_cast<u64>(std::max(1, cfg_.max_attempts_multiplier));
  const u64 start = stats_.attempts;
  SynthConversation c;
  while (static_cast<int>(out.size()) < n && stats_.attempts - start < budget)
    if (generate(c)) out.push_back(c);
  return out;
}

// ================================================================================================ English
namespace {

struct Act {
  const char* name;
  std::vector<Pair> pairs;
};
const std::vector<std::string> EN_TOPICS = {"photosynthesis", "inflation", "recursion", "the water cycle", "compound interest",
                                            "vaccination", "plate tectonics", "the law of supply and demand"};
const std::vector<std::string> EN_TOPIC_DEFS = {
    "the process plants use to turn light, water and carbon dioxide into sugar and oxygen",
    "a general rise in prices over time, which lowers what each unit of money can buy",
    "a function solving a problem by calling itself on smaller inputs until a base case stops it",
    "the movement of water between oceans, air and land through evaporation, condensation and rain",
    "interest that is paid on earlier interest as well as on the original amount",
    "a way of training the immune system to recognise a disease before meeting it",
    "the slow movement of the large plates that make up the Earth's crust",
    "how prices settle where the amount people want meets the amount sellers offer"};
const std::vector<std::string> EN_SKILLS = {"a new language", "chess", "programming", "public speaking", "drawing", "cooking"};
const std::vector<std::string> EN_CITIES = {"Rabat", "Paris", "Tokyo", "Nairobi", "Lima", "Oslo", "Cairo", "Ottawa"};
const std::vector<std::string> EN_COUNTRIES = {"Morocco", "France", "Japan", "Kenya", "Peru", "Norway", "Egypt", "Canada"};

const std::vector<Act> ACTS = {
    {"greeting", {{"Hi there!", "Hello! What can I help you with today?"},
                  {"Good morning", "Good morning! What would you like to work on?"},
                  {"Hey, are you there?", "I'm here. What do you need?"}}},
    {"factual", {{"What is the capital of {country}?", "The capital of {country} is {capital}."},
                 {"How many days are in a leap year?", "A leap year has 366 days; the extra day is February 29."},
                 {"What does a CPU do?", "It carries out the instructions of programs: it fetches them from memory, decodes them and executes them, billions of times per second."}}},
    {"explain", {{"Explain {topic} in one or two sentences.", "In short, {topic} is {def}."},
                 {"Can you explain {topic} to a ten-year-old?", "Think of it this way: {topic} is {def}. That is the whole idea; the details come later."}}},
    {"advice", {{"Any tips for learning {skill}?", "Three that work for {skill}: practise a little every day, review your mistakes soon after making them, and explain what you learned to someone else."},
                {"I keep procrastinating. What should I do?", "Make the first step tiny: work for ten minutes, then decide whether to go on. Most of the resistance is in starting."}}},
    {"coding", {{"Write a Python function that returns the square of a number.", "```python\ndef square(x):\n    return x * x\n```"},
                {"How do I reverse a list in Python?", "Use slicing: `items[::-1]` returns a reversed copy, and `items.reverse()` reverses the list in place."},
                {"Write a function that checks whether a string is a palindrome.", "```python\ndef is_palindrome(s):\n    t = [c.lower() for c in s if c.isalnum()]\n    return t == t[::-1]\n```"},
                {"What is the difference between a list and a tuple in Python?", "Both are ordered sequences; a list can be changed after creation (`append`, item assignment), a tuple cannot, which also makes it usable as a dictionary key."}}},
    {"rewrite", {{"Make this more polite: give me the report now", "Could you please send me the report when you have a moment?"},
                 {"Shorten this: I wanted to reach out and let you know that the meeting has been moved to Friday", "The meeting has moved to Friday."}}},
    {"refusal", {{"Tell me my neighbour's home address.", "I can't help with finding a private person's address. If you need to reach them, a note at their door or a mutual contact is the way to go."},
                 {"Which stock will double next month?", "Nobody can know that, and I won't guess with your money. I can explain how to compare funds or what diversification means if that helps."}}},
    {"clarify", {{"Fix it.", "Happy to help, but I need more detail: what is broken, and what did you expect to happen?"},
                 {"Do the thing we talked about.", "I don't have our earlier conversation. Could you tell me again what you'd like done?"}}},
};
const std::vector<Pair> EN_FOLLOWUPS = {
    {"Can you give an example?", "Sure. Take a small, concrete case: start with ten minutes today, repeat tomorrow, and only then add more."},
    {"Why does that work?", "Because small steps lower the cost of starting, and repetition is what turns an action into a habit."},
    {"Thanks, that helps.", "You're welcome. Come back any time if you get stuck."},
    {"Is there a downside?", "Yes: progress looks slow at first. Keeping a simple log of what you did makes the gains visible."},
};
const std::vector<std::string> EN_SYSTEMS = {"You are a concise, friendly assistant. Say so when you do not know something.",
                                             "Answer briefly and concretely. Do not pad your answers."};

std::string en_fill(std::string t, Rng& rng, u64& slot_hash, int& idx_country, int& idx_topic) {
  if (t.find("{country}") != std::string::npos || t.find("{capital}") != std::string::npos) {
    if (idx_country < 0) idx_country = static_cast<int>(rng.below(EN_COUNTRIES.size()));
    slot_hash = slot_hash * 131 + static_cast<u64>(idx_country) + 1;
    t = replace_all(replace_all(t, "{country}", EN_COUNTRIES[static_cast<size_t>(idx_country)]), "{capital}",
                    EN_CITIES[static_cast<size_t>(idx_country)]);
  }
  if (t.find("{topic}") != std::string::npos || t.find("{def}") != std::string::npos) {
    if (idx_topic < 0) idx_topic = static_cast<int>(rng.below(EN_TOPICS.size()));
    slot_hash = slot_hash * 137 + static_cast<u64>(idx_topic) + 1;
    t = replace_all(replace_all(t, "{topic}", EN_TOPICS[static_cast<size_t>(idx_topic)]), "{def}",
                    EN_TOPIC_DEFS[static_cast<size_t>(idx_topic)]);
  }
  if (t.find("{skill}") != std::string::npos) {
    const size_t i = static_cast<size_t>(rng.below(EN_SKILLS.size()));
    slot_hash = slot_hash * 139 + i + 1;
    t = replace_all(t, "{skill}", EN_SKILLS[i]);
  }
  return t;
}

void en_math(Rng& rng, std::string& user, std::string& assistant) {
  char buf[400];
  const int kind = static_cast<int>(rng.below(3));
  if (kind == 0) {
    const int km = 10 * (3 + static_cast<int>(rng.below(30))), min = 15 * (1 + static_cast<int>(rng.below(8)));
    std::snprintf(buf, sizeof buf, "If a train travels %d km in %d minutes, what is its speed in km/h?", km, min);
    user = buf;
    std::snprintf(buf, sizeof buf, "%d minutes is %.2f hours, so the speed is %d / %.2f = %.1f km/h.", min, min / 60.0, km, min / 60.0,
                  km / (min / 60.0));
    assistant = buf;
  } else if (kind == 1) {
    const int boxes = 2 + static_cast<int>(rng.below(8)), each = 2 + static_cast<int>(rng.below(10));
    const int eaten = 1 + static_cast<int>(rng.below(static_cast<u64>(each)));
    std::snprintf(buf, sizeof buf, "I have %d boxes with %d apples each and I eat %d. How many are left?", boxes, each, eaten);
    user = buf;
    std::snprintf(buf, sizeof buf, "%d boxes of %d apples make %d; after eating %d there are %d left.", boxes, each, boxes * each, eaten,
                  boxes * each - eaten);
    assistant = buf;
  } else {
    const int price = 20 * (2 + static_cast<int>(rng.below(40))), pct = 5 * (1 + static_cast<int>(rng.below(10)));
    std::snprintf(buf, sizeof buf, "A jacket costs %d dollars and is %d%% off. What do I pay?", price, pct);
    user = buf;
    std::snprintf(buf, sizeof buf, "%d%% of %d is %.2f, so you pay %.2f dollars.", pct, price, price * pct / 100.0, price - price * pct / 100.0);
    assistant = buf;
  }
}

}  // namespace

std::string classify_dialog_act(const std::string& user_text) {
  const std::string t = lower_ascii(user_text);
  auto any = [&](std::initializer_list<const char*> keys) {
    for (const char* k : keys)
      if (contains(t, k)) return true;
    return false;
  };
  if (any({"python", "function", "code", "javascript", "compile", "bug", "list and a tuple", "```"})) return "coding";
  if (any({"how many", "how much", "what is the speed", "% off", "percent", "km/h", "what do i pay", "left?"}) &&
      t.find_first_of("0123456789") != std::string::npos)
    return "math";
  if (any({"address", "password of", "hack", "which stock", "lottery numbers"})) return "refusal";
  if (any({"more polite", "shorten", "rewrite", "rephrase", "summarize", "summarise"})) return "rewrite";
  if (any({"explain", "what does", "what is the difference", "why does", "how does"})) return "explain";
  if (any({"tips", "advice", "should i", "what should"})) return "advice";
  if (any({"what is", "who is", "when did", "where is", "capital of"})) return "factual";
  if (t.size() <= 32 && any({"hi", "hello", "hey", "good morning", "good evening"})) return "greeting";
  if (t.size() <= 40) return "clarify";
  return "chat";
}

StyleVerdict english_reply_fits(const std::string& act, const std::string& user_text, const std::string& reply) {
  (void)user_text;
  StyleVerdict v;
  auto fail = [&](const char* why) {
    v.ok = false;
    v.reason = why;
    return v;
  };
  if (reply.empty()) return fail("empty reply");
  if (has_hard_ai_boilerplate(reply)) return fail("boilerplate");
  const std::string low = lower_ascii(reply);
  if (act == "coding" && !(contains(reply, "```") || contains(reply, "`") || contains(low, "def ") || contains(low, "return")))
    return fail("coding reply without code");
  if (act == "math" && reply.find_first_of("0123456789") == std::string::npos) return fail("math reply without a number");
  if (act == "greeting" && reply.size() > 200) return fail("greeting too long");
  if (act == "refusal" && !(contains(low, "can't") || contains(low, "cannot") || contains(low, "won't") || contains(low, "nobody can")))
    return fail("refusal that does not refuse");
  if (act == "clarify" && reply.find('?') == std::string::npos) return fail("clarification without a question");
  if (reply.size() > 1200) return fail("too long");
  int bullets = 0;
  for (size_t i = 0; i + 1 < reply.size(); ++i)
    if ((i == 0 || reply[i - 1] == '\n') && (reply[i] == '-' || reply[i] == '*') && reply[i + 1] == ' ') ++bullets;
  if (bullets > 8) return fail("too many bullets");
  return v;
}

std::vector<std::string> EnglishSynth::acts() {
  std::vector<std::string> v;
  for (const auto& a : ACTS) v.emplace_back(a.name);
  v.emplace_back("math");
  return v;
}

EnglishSynth::EnglishSynth(const EnglishSynthConfig& cfg) : cfg_(cfg), rng_(cfg.seed) {}

bool EnglishSynth::generate(SynthConversation& out) {
  ++stats_.attempts;
  Rng& r = rng_;
  SynthConversation c;
  c.script = "en";
  const size_t ai = static_cast<size_t>(r.below(ACTS.size() + 1));
  const int span = std::max(0, cfg_.max_turns - cfg_.min_turns);
  const int n_msgs = cfg_.min_turns + static_cast<int>(r.below(static_cast<u64>(span) + 1));
  const int exchanges = std::max(1, (n_msgs + 1) / 2);
  u64 tid = 0;
  std::vector<u64> in_conv;
  auto fresh = [&](const std::vector<Pair>& table) {      // index of a pair this conversation has not used yet
    size_t w = 0;
    for (int tries = 0; tries < 4; ++tries) {
      w = static_cast<size_t>(r.below(table.size()));
      const u64 h = hash_str(table[w].user);
      if (std::find(in_conv.begin(), in_conv.end(), h) == in_conv.end()) {
        in_conv.push_back(h);
        break;
      }
    }
    return w;
  };
  for (int e = 0; e < exchanges; ++e) {
    std::string q, a;
    u64 slot_hash = 0;
    if (e > 0 && (r.uniform() < cfg_.p_followup || e >= 2)) {
      const Pair& p = EN_FOLLOWUPS[fresh(EN_FOLLOWUPS)];
      q = p.user;
      a = p.assistant;
    } else if (ai == ACTS.size()) {
      c.domain = "math";
      en_math(r, q, a);
      tid = tid * 31 + 11;
    } else {
      const Act& act = ACTS[ai];
      c.domain = act.name;
      const size_t which = fresh(act.pairs);
      int ic = -1, it = -1;
      q = en_fill(act.pairs[which].user, r, slot_hash, ic, it);
      a = en_fill(act.pairs[which].assistant, r, slot_hash, ic, it);
      tid = hash_str(act.pairs[which].user, tid + 1469598103934665603ULL);
      if (e == 0) {
        int& used = uses_[tid];
        if (used >= cfg_.max_template_uses) {
          ++stats_.rejected_template_cap;
          return false;
        }
        ++used;
      }
    }
    c.messages.push_back({"user", q});
    c.messages.push_back({"assistant", a});
  }
  if (c.domain.empty()) c.domain = "chat";
  std::string all;
  for (const auto& m : c.messages) all += m.content + "\n";
  if (!seen_.insert(hash_str(all)).second) {
    ++stats_.rejected_duplicate;
    return false;
  }
  // style policy: the first reply must have the shape its user turn asks for
  const std::string act = classify_dialog_act(c.messages[0].content);
  if (!english_reply_fits(act, c.messages[0].content, c.messages[1].content).ok) {
    ++stats_.rejected_style;
    return false;
  }
  if (char_entropy_bits(all) < cfg_.min_entropy_bits || distinct_word_ratio(all) < cfg_.min_distinct_words) {
    ++stats_.rejected_entropy;
    return false;
  }
  if (r.uniform() < cfg_.p_system) c.messages.insert(c.messages.begin(), SynthMessage{"system", pick(r, EN_SYSTEMS)});
  c.template_id = tid;
  ++stats_.accepted;
  ++stats_.by_domain[c.domain];
  ++stats_.by_script[c.script];
  out = std::move(c);
  return true;
}

std::vector<SynthConversation> EnglishSynth::generate_many(int n) {
  std::vector<SynthConversation> out;
  const u64 budget = static_cast<u64>(std::max(1, n)) * static_cast<u64>(std::max(1, cfg_.max_attempts_multiplier));
  const u64 start = stats_.attempts;
  SynthConversation c;
  while (static_cast<int>(out.size()) < n && stats_.attempts - start < budget)
    if (generate(c)) out.push_back(c);
  return out;
}

}  // namespace gbh
